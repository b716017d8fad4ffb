// Generic exact-fp32 split decode kernel: any D <= 256 (multiple of 8), any group, GQA width
// up to 16, no alignment requirement on block starts.  It is the path for shapes the
// tensor-core kernel does not cover, and the CUDA-core baseline the tensor-core kernel is
// measured against.
//
// One CTA owns a slice of consecutive blocks of one cache row (the split-K of
// geodesia_kv_cuda/mixed_attn.cu:58-65) and every query head of that row's GQA group.
// Per block: dequantise K and V into shared fp32 tiles (coalesced reads, one pass over the
// bytes for the whole group), score 64 tokens x rep heads, one warp per head does the online
// softmax update, then every thread owns (head, channel) output pairs for the V product.
#pragma once

#include "gkv_common.cuh"

namespace gkv {

struct DecodeParams {
    const float* q;
    const uint8_t* data;
    const int64_t* offs;
    const __half* klo;
    const __half* kstep;
    const __half* vlo;
    const __half* vstep;
    const int32_t* level;
    const int32_t* valid;
    float* part;      // (rows, nsplit, rep, D+2): m, l, o[D]
    int B, Hq, Hkv, D, nb, group, G, gv, rep;
    int nsplit, bps;
    int per_row_meta; // 0: one metadata row shared by all cache rows
    int64_t stride_bh;
};

constexpr int kGenThreads = 256;

__device__ __forceinline__ uint32_t load_u32_any(const uint8_t* p, bool aligned4) {
    if (aligned4) return *reinterpret_cast<const uint32_t*>(p);
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

// Dequantise 4 consecutive elements (same token, channels d..d+3) of one plane.
__device__ __forceinline__ void dequant4(const uint8_t* __restrict__ plane, int lv, int e, bool al,
                                         float (&x)[4]) {
    if (lv == 16) {
        const uint32_t w0 = load_u32_any(plane + (size_t)e * 2, al);
        const uint32_t w1 = load_u32_any(plane + (size_t)e * 2 + 4, al);
        x[0] = __uint_as_float(w0 << 16);
        x[1] = __uint_as_float(w0 & 0xffff0000u);
        x[2] = __uint_as_float(w1 << 16);
        x[3] = __uint_as_float(w1 & 0xffff0000u);
    } else if (lv == 8) {
        const uint32_t w = load_u32_any(plane + e, al);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = (float)((w >> (8 * i)) & 0xffu);
    } else if (lv == 4) {
        const uint32_t w = (uint32_t)plane[e / 2] | ((uint32_t)plane[e / 2 + 1] << 8);
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = (float)((w >> (4 * i)) & 0xfu);
    } else {
        const uint32_t w = plane[e / 4];
#pragma unroll
        for (int i = 0; i < 4; ++i) x[i] = (float)((w >> (2 * i)) & 0x3u);
    }
}

__global__ void __launch_bounds__(kGenThreads) decode_generic_kernel(DecodeParams p) {
    extern __shared__ float smem[];
    const int D = p.D, rep = p.rep, KS = D + 1;
    float* sq = smem;                      // rep * D
    float* sk = sq + rep * D;              // 64 * (D+1)
    float* sv = sk + kP * KS;              // 64 * D
    float* sw = sv + kP * D;               // rep * 64
    float* sm = sw + rep * kP;             // rep: running max
    float* sl = sm + rep;                  // rep: running sum
    float* srs = sl + rep;                 // rep: rescale of this block

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sp = blockIdx.x, row = blockIdx.y;
    const int b = row / p.Hkv, hk = row % p.Hkv;
    const int mrow = p.per_row_meta ? row : 0;
    const int64_t* offs = p.offs + (size_t)mrow * p.nb;
    const int32_t* level = p.level + (size_t)mrow * p.nb;
    const int32_t* valid = p.valid + (size_t)mrow * p.nb;
    const uint8_t* base = p.data + (size_t)row * p.stride_bh;
    const float* q = p.q + ((size_t)b * p.Hq + (size_t)hk * rep) * D;

    for (int i = tid; i < rep * D; i += kGenThreads) sq[i] = q[i];
    if (tid < rep) { sm[tid] = -INFINITY; sl[tid] = 0.f; srs[tid] = 0.f; }

    constexpr int kMaxAcc = 16;            // rep * D / 256 <= 16 * 256 / 256
    float acc[kMaxAcc];
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) acc[i] = 0.f;
    __syncthreads();

    const int b_lo = sp * p.bps, b_hi = min(p.nb, b_lo + p.bps);
    for (int blk = b_lo; blk < b_hi; ++blk) {
        const int lv = level[blk];
        const int nvalid = min(valid[blk], kP);
        if (nvalid <= 0 || !level_ok(lv)) continue;   // uniform across the CTA
        const uint8_t* kb = base + offs[blk];
        const uint8_t* vb = kb + half_bytes(lv, D);
        const bool al = ((reinterpret_cast<uintptr_t>(kb) & 3) == 0);

        // ---- dequantise into the tiles --------------------------------------------
        if (lv == 1) {
            for (int e = tid; e < kP * D; e += kGenThreads) {
                const int j = e / D, d = e - j * D;
                sk[j * KS + d] = half_bits_to_float(reinterpret_cast<const uint16_t*>(kb)[d]);
                sv[j * D + d] = half_bits_to_float(reinterpret_cast<const uint16_t*>(vb)[d]);
            }
        } else {
            const size_t kso = (((size_t)row * p.nb + blk) * p.G) * D;
            const size_t vso = (((size_t)row * p.nb + blk) * kP) * p.gv;
            for (int e = tid * 4; e < kP * D; e += kGenThreads * 4) {
                const int j = e / D, d = e - j * D;
                float xk[4], xv[4];
                dequant4(kb, lv, e, al, xk);
                dequant4(vb, lv, e, al, xv);
                if (lv != 16) {
                    const size_t ks = kso + (size_t)(j / p.group) * D + d;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const size_t vs = vso + (size_t)j * p.gv + (d + i) / p.group;
                        xk[i] = xk[i] * __half2float(p.kstep[ks + i]) + __half2float(p.klo[ks + i]);
                        xv[i] = xv[i] * __half2float(p.vstep[vs]) + __half2float(p.vlo[vs]);
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    sk[j * KS + d + i] = xk[i];
                    sv[j * D + d + i] = xv[i];
                }
            }
        }
        __syncthreads();

        // ---- scores: one (head, token) pair per thread ------------------------------
        for (int pr = tid; pr < rep * kP; pr += kGenThreads) {
            const int h = pr >> 6, j = pr & 63;
            float s = -INFINITY;
            if (j < nvalid) {
                s = 0.f;
                const float* qq = sq + h * D;
                const float* kk = sk + j * KS;
#pragma unroll 8
                for (int d = 0; d < D; ++d) s = fmaf(qq[d], kk[d], s);
            }
            sw[pr] = s;
        }
        __syncthreads();

        // ---- online softmax: warp w updates heads w, w+8, ... ------------------------
        for (int h = warp; h < rep; h += kGenThreads / 32) {
            const float s0 = sw[h * kP + lane], s1 = sw[h * kP + lane + 32];
            float mb = fmaxf(s0, s1);
#pragma unroll
            for (int o = 16; o; o >>= 1) mb = fmaxf(mb, __shfl_xor_sync(0xffffffffu, mb, o));
            const float mold = sm[h];
            const float mnew = fmaxf(mold, mb);
            const float w0 = (s0 == -INFINITY) ? 0.f : expf(s0 - mnew);
            const float w1 = (s1 == -INFINITY) ? 0.f : expf(s1 - mnew);
            float lb = w0 + w1;
#pragma unroll
            for (int o = 16; o; o >>= 1) lb += __shfl_xor_sync(0xffffffffu, lb, o);
            sw[h * kP + lane] = w0;
            sw[h * kP + lane + 32] = w1;
            if (lane == 0) {
                const float rs = (mold == -INFINITY) ? 0.f : expf(mold - mnew);
                sl[h] = sl[h] * rs + lb;
                sm[h] = mnew;
                srs[h] = rs;
            }
        }
        __syncthreads();

        // ---- V product: thread owns (head, channel) pairs ------------------------------
#pragma unroll
        for (int i = 0; i < kMaxAcc; ++i) {
            const int pr = tid + i * kGenThreads;
            if (pr < rep * D) {
                const int h = pr / D, d = pr - h * D;
                float a = acc[i] * srs[h];
                const float* ww = sw + h * kP;
                for (int j = 0; j < nvalid; ++j) a = fmaf(ww[j], sv[j * D + d], a);
                acc[i] = a;
            }
        }
        __syncthreads();
    }

    float* part = p.part + ((size_t)row * p.nsplit + sp) * rep * (D + 2);
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) {
        const int pr = tid + i * kGenThreads;
        if (pr < rep * D) {
            const int h = pr / D, d = pr - h * D;
            part[(size_t)h * (D + 2) + 2 + d] = acc[i];
        }
    }
    if (tid < rep) {
        part[(size_t)tid * (D + 2) + 0] = sm[tid];
        part[(size_t)tid * (D + 2) + 1] = sl[tid];
    }
}

inline size_t decode_generic_smem(int rep, int D) {
    return sizeof(float) * ((size_t)rep * D + (size_t)kP * (D + 1) + (size_t)kP * D + (size_t)rep * kP + 3 * rep);
}

}  // namespace gkv
