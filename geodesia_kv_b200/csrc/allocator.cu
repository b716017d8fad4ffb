// Rate-distortion rung allocator and its distortion table, one CTA per cache row.
//
// The reference (geodesia_kv/policies.py:810-868) sorts all 4*nb marginal-cost ratios and
// bisects over the sorted array for the first candidate threshold whose allocation fits the
// bit budget.  The feasible thresholds form an up-set of the candidate values, so the same
// threshold is found without a sort by bisecting over the order-preserving integer image of
// fp32: the smallest feasible key inside [min candidate, max candidate] is that candidate,
// the min candidate when every threshold fits, the max candidate when none does.  The
// allocation at a threshold takes, per block, the longest prefix (from ladder step 0) of
// available steps whose ratio is <= threshold, so a block that has already left rung 16
// never moves again — the reference's behaviour, kept on purpose.
#include "gkv_common.cuh"

namespace gkv {

constexpr int kAllocThreads = 512;

__device__ __forceinline__ uint32_t float_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct AllocParams {
    const float* mass; const float* E; const int32_t* idx; const uint8_t* hot;
    const double* target_bits; float* ratio; int32_t* tgt;
    float bits[5];
    float mass_power;
    int nb;
    const int32_t* nb_of;      // optional: blocks in use per problem (rows of a ragged batch); the rest keep their rung
};

template <typename T, typename Op>
__device__ T block_reduce(T v, Op op, T* scratch) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, o));
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    T r = scratch[0];
    for (int w = 1; w < kAllocThreads / 32; ++w) r = op(r, scratch[w]);
    return r;
}

// Ladder index a block lands on at threshold lam (the prefix rule).
__device__ __forceinline__ int landing(const float* __restrict__ r4, int idx, bool hot, float lam) {
    int pref = 0;
#pragma unroll
    for (int s = 0; s < 4; ++s) {
        const bool ok = (r4[s] <= lam) && (s >= idx) && !hot;
        if (ok && pref == s) pref = s + 1;
    }
    return min(idx + pref, 4);
}

__global__ void __launch_bounds__(kAllocThreads) allocate_kernel(AllocParams p) {
    __shared__ double sd[kAllocThreads / 32];
    __shared__ uint32_t su[kAllocThreads / 32];
    const int prob = blockIdx.x, tid = threadIdx.x;
    const int nb_all = p.nb;
    const int nb = p.nb_of ? max(0, min(nb_all, p.nb_of[prob])) : nb_all;
    const float* mass = p.mass + (size_t)prob * nb_all;
    const float* E = p.E + (size_t)prob * nb_all * 5;
    const int32_t* idx = p.idx + (size_t)prob * nb_all;
    const uint8_t* hot = p.hot + (size_t)prob * nb_all;
    float* ratio = p.ratio + (size_t)prob * nb_all * 4;
    int32_t* tgt = p.tgt + (size_t)prob * nb_all;
    for (int b = nb + tid; b < nb_all; b += kAllocThreads) tgt[b] = idx[b];
    const float big = 3.4028234663852886e38f / 4.0f;

    uint32_t kmin = 0xffffffffu, kmax = 0u;
    for (int b = tid; b < nb; b += kAllocThreads) {
        float mc = fmaxf(mass[b], 1e-12f);
        if (p.mass_power != 1.0f) mc = powf(mc, p.mass_power);
        float dmg[5];
#pragma unroll
        for (int c = 0; c < 5; ++c) dmg[c] = __fmul_rn(mc, E[b * 5 + c]);
        const int id = idx[b];
        const bool h = hot[b] != 0;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            const float gain = fmaxf(__fsub_rn(p.bits[s], p.bits[s + 1]), 1e-9f);
            const float cost = __fsub_rn(dmg[s + 1], dmg[s]);
            const float r = ((s >= id) && !h) ? __fdiv_rn(cost, gain) : big;
            ratio[b * 4 + s] = r;
            const uint32_t k = float_key(r);
            kmin = min(kmin, k);
            kmax = max(kmax, k);
        }
    }
    kmin = block_reduce(kmin, [](uint32_t a, uint32_t b) { return a < b ? a : b; }, su);
    kmax = block_reduce(kmax, [](uint32_t a, uint32_t b) { return a > b ? a : b; }, su);
    __syncthreads();   // ratio[] written by this CTA is read back below
    if (nb == 0) return;

    const float target = (float)p.target_bits[prob];   // fp32 comparison, as torch does
    auto fits = [&](float lam) -> bool {
        double tot = 0.0;
        for (int b = tid; b < nb; b += kAllocThreads)
            tot += (double)p.bits[landing(ratio + b * 4, idx[b], hot[b] != 0, lam)];
        tot = block_reduce(tot, [](double a, double b) { return a + b; }, sd);
        return !((float)tot > target);
    };

    uint32_t lo = kmin, hi = kmax;
    if (fits(key_float(kmax))) {
        while (lo < hi) {
            const uint32_t mid = lo + ((hi - lo) >> 1);
            if (fits(key_float(mid))) hi = mid;
            else lo = mid + 1;
        }
    }
    const float lam = key_float(hi);
    for (int b = tid; b < nb; b += kAllocThreads)
        tgt[b] = landing(ratio + b * 4, idx[b], hot[b] != 0, lam);
}

// ---- distortion table (policies.py:774-808) from rung-16 blocks of the packed cache ------
struct DistParams {
    const uint8_t* data; const int64_t* offs; const int32_t* level; float* E;
    int nb, D, group, per_row_meta;
    float value_weight;
    int64_t stride_bh;
};

constexpr int kDistThreads = 256;

__global__ void __launch_bounds__(kDistThreads) distortion_kernel(DistParams p) {
    extern __shared__ float smem[];
    const int D = p.D, tid = threadIdx.x;
    const int kg = min(p.group, kP), vg = min(p.group, D);
    const int G = kP / kg, gv = D / vg;
    // tile rows are padded by one float: several passes below walk a row per thread, and rows an
    // exact multiple of 32 floats apart would all sit in one bank
    const int ld = D + 1;
    float* sk = smem;                    // [64][ld]
    float* sv = sk + kP * ld;            // [64][ld]
    float* rk = sv + kP * ld;            // [G][D]   K ranges
    float* rv = rk + G * D;              // [64][gv] V ranges
    float* mean = rv + kP * gv;          // [2][D]
    float* rad = mean + 2 * D;           // [2][64]
    float* ek = rad + 2 * kP;            // [3][G]
    float* ev = ek + 3 * G;              // [3][64]
    const int blk = blockIdx.x, row = blockIdx.y;
    const int mrow = p.per_row_meta ? row : 0;
    const size_t mi = (size_t)mrow * p.nb + blk;
    float* Eo = p.E + ((size_t)row * p.nb + blk) * 5;
    if (p.level[mi] != 16) {
        if (tid < 5) Eo[tid] = 0.f;
        return;
    }
    const uint16_t* kb = reinterpret_cast<const uint16_t*>(p.data + (size_t)row * p.stride_bh + p.offs[mi]);
    const uint16_t* vb = kb + kP * D;
    if ((reinterpret_cast<uintptr_t>(kb) & 15) == 0) {
        const uint4* k8 = reinterpret_cast<const uint4*>(kb);
        const uint4* v8 = reinterpret_cast<const uint4*>(vb);
        for (int e8 = tid; e8 < kP * D / 8; e8 += kDistThreads) {        // D % 8 == 0: a load stays inside a row
            const int t = (8 * e8) / D, d = 8 * e8 - t * D;
            const uint4 a = k8[e8], b = v8[e8];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                sk[t * ld + d + 2 * i] = bf16_bits_to_float(aw[i] & 0xffffu);
                sk[t * ld + d + 2 * i + 1] = bf16_bits_to_float(aw[i] >> 16);
                sv[t * ld + d + 2 * i] = bf16_bits_to_float(bw[i] & 0xffffu);
                sv[t * ld + d + 2 * i + 1] = bf16_bits_to_float(bw[i] >> 16);
            }
        }
    } else {
        for (int e = tid; e < kP * D; e += kDistThreads) {
            const int t = e / D, d = e - t * D;
            sk[t * ld + d] = bf16_bits_to_float(kb[e]);
            sv[t * ld + d] = bf16_bits_to_float(vb[e]);
        }
    }
    __syncthreads();
    for (int u = tid; u < G * D; u += kDistThreads) {
        const int tg = u / D, d = u - tg * D;
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < kg; ++i) { const float x = sk[(tg * kg + i) * ld + d]; lo = fminf(lo, x); hi = fmaxf(hi, x); }
        rk[u] = __fsub_rn(hi, lo);
    }
    for (int u = tid; u < kP * gv; u += kDistThreads) {
        const int t = u / gv, cg = u - t * gv;
        float lo = INFINITY, hi = -INFINITY;
        for (int i = 0; i < vg; ++i) { const float x = sv[t * ld + cg * vg + i]; lo = fminf(lo, x); hi = fmaxf(hi, x); }
        rv[u] = __fsub_rn(hi, lo);
    }
    for (int u = tid; u < 2 * D; u += kDistThreads) {
        const float* src = u < D ? sk + u : sv + (u - D);
        float s = 0.f;
        for (int t = 0; t < kP; ++t) s = __fadd_rn(s, src[t * ld]);
        mean[u] = __fdiv_rn(s, (float)kP);
    }
    __syncthreads();
    for (int u = tid; u < 2 * kP; u += kDistThreads) {
        const int which = u / kP, t = u - which * kP;
        const float* src = (which ? sv : sk) + t * ld;
        const float* mu = mean + which * D;
        float s = 0.f;
        for (int d = 0; d < D; ++d) { const float x = __fsub_rn(src[d], mu[d]); s = __fadd_rn(s, __fmul_rn(x, x)); }
        rad[u] = __fsqrt_rn(s);
    }
    for (int u = tid; u < 3 * G; u += kDistThreads) {
        const int li = u / G, tg = u - li * G;
        const float den = 2.0f * (float)((1 << (8 >> li)) - 1);
        float s = 0.f;
        for (int d = 0; d < D; ++d) { const float x = __fdiv_rn(rk[tg * D + d], den); s = __fadd_rn(s, __fmul_rn(x, x)); }
        ek[u] = __fsqrt_rn(s);
    }
    for (int u = tid; u < 3 * kP; u += kDistThreads) {
        const int li = u / kP, t = u - li * kP;
        const float den = 2.0f * (float)((1 << (8 >> li)) - 1);
        float s = 0.f;
        for (int cg = 0; cg < gv; ++cg) {
            const float x = __fdiv_rn(rv[t * gv + cg], den);
            s = __fadd_rn(s, __fmul_rn(__fmul_rn(x, x), (float)vg));
        }
        ev[u] = __fsqrt_rn(s);
    }
    __syncthreads();
    if (tid < 5) {
        float a = 0.f, b = 0.f;
        if (tid == 4) {
            for (int t = 0; t < kP; ++t) { a = fmaxf(a, rad[t]); b = fmaxf(b, rad[kP + t]); }
        } else if (tid > 0) {
            const int li = tid - 1;
            for (int tg = 0; tg < G; ++tg) a = fmaxf(a, ek[li * G + tg]);
            for (int t = 0; t < kP; ++t) b = fmaxf(b, ev[li * kP + t]);
        }
        Eo[tid] = __fadd_rn(a, __fmul_rn(p.value_weight, b));
    }
}

}  // namespace gkv

extern "C" {

int gkv_allocate(const float* mass, const float* E, const int32_t* idx, const uint8_t* hot,
                 const float* bits_host, const double* target_bits, float mass_power, float* ratio,
                 int32_t* tgt_idx, int problems, int nb, void* stream) {
    return gkv_allocate_ragged(mass, E, idx, hot, bits_host, target_bits, mass_power, ratio, tgt_idx, nullptr,
                               problems, nb, stream);
}

int gkv_allocate_ragged(const float* mass, const float* E, const int32_t* idx, const uint8_t* hot,
                        const float* bits_host, const double* target_bits, float mass_power, float* ratio,
                        int32_t* tgt_idx, const int32_t* nb_of, int problems, int nb, void* stream) {
    using namespace gkv;
    if (problems <= 0 || nb < 0) return GKV_E_SHAPE;
    if (!bits_host) return GKV_E_NULL;
    if (nb == 0) return GKV_OK;
    if (!mass || !E || !idx || !hot || !target_bits || !ratio || !tgt_idx) return GKV_E_NULL;
    AllocParams p;
    p.mass = mass; p.E = E; p.idx = idx; p.hot = hot; p.target_bits = target_bits; p.ratio = ratio;
    p.tgt = tgt_idx; p.mass_power = mass_power; p.nb = nb; p.nb_of = nb_of;
    for (int i = 0; i < 5; ++i) p.bits[i] = bits_host[i];
    allocate_kernel<<<problems, kAllocThreads, 0, (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

int gkv_block_distortion(const uint8_t* data, const int64_t* offs, const int32_t* level, float* E, int rows,
                         int nb, int D, int block, int group, float value_weight, int64_t stride_bh,
                         int meta_rows, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (rows <= 0 || nb <= 0 || D <= 0 || D > kMaxD || D % 8 || group <= 0) return GKV_E_SHAPE;
    if (kP % min(group, kP) || D % min(group, D)) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (!data || !offs || !level || !E) return GKV_E_NULL;
    DistParams p;
    p.data = data; p.offs = offs; p.level = level; p.E = E; p.nb = nb; p.D = D; p.group = group;
    p.per_row_meta = meta_rows != 1; p.value_weight = value_weight; p.stride_bh = stride_bh;
    const int kg = min(group, kP), vg = min(group, D);
    const int G = kP / kg, gv = D / vg;
    const size_t smem = sizeof(float) * ((size_t)2 * kP * (D + 1) + (size_t)G * D + (size_t)kP * gv + 2 * D + 2 * kP + 3 * G + 3 * kP);
    const size_t smem_max = sizeof(float) * ((size_t)2 * kP * (kMaxD + 1) + (size_t)kP * kMaxD + (size_t)kP * kMaxD + 2 * kMaxD + 2 * kP + 3 * kP + 3 * kP);
    GKV_CUDA_TRY(cudaFuncSetAttribute(distortion_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      (int)(smem_max > 227 * 1024 ? 227 * 1024 : smem_max)));
    if (smem > 227 * 1024) return GKV_E_SHAPE;
    distortion_kernel<<<dim3(nb, rows), kDistThreads, smem, (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

}  // extern "C"
