// Decode attention over the packed cache: planning, the LSE combine and the C ABI.
#include <stdlib.h>
#include <string.h>

#include "decode_generic.cuh"
#include "decode_mma.cuh"

namespace gkv {

int g_last_cuda_error = 0;

// ---- LSE merge of split records -----------------------------------------------------------
// Records are D+2 floats [m, l, o[D]].  Record s of output row r lives at
//   rec + r_base(r) + s * stride_s.
// Follows geodesia_kv_cuda/mixed_attn.cu:171-200 (splits with m = -inf are skipped, the
// denominator clamps at 1e-20); `normalise == 0` writes the merged record instead of o/l.
struct CombineParams {
    const float* rec;
    float* out;
    int parts, D;
    int rep, nsplit;     // internal layout (rows, nsplit, rep, D+2) when rep > 0
    int64_t stride_s;    // external layout (parts, rows, D+2) when rep == 0
    int normalise;
    const int* status;   // when non-null and non-zero the producing kernel gave up: poison the output
    int segs;            // > 1: blockIdx.y merges records [y*per_seg, (y+1)*per_seg) into record y of
    int per_seg;         //      an external-layout (segs, rows, D+2) buffer (normalise must be 0)
};

constexpr int kCombineThreads = 256;

// One CTA per output row.  The records of a row are shared out over the 8 warps (record s goes
// to warp s mod 8, whose lanes read it coalesced), each warp keeps a running (m, l, o) of its
// records, and the 8 states are merged through shared memory — the same recurrence at both levels.
__global__ void __launch_bounds__(kCombineThreads) combine_kernel(CombineParams p) {
    __shared__ float sm_m[8], sm_l[8], sm_o[8][kMaxD];
    const int orow = blockIdx.x, D = p.D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* base;
    int64_t stride;
    if (p.rep > 0) {
        const int row = orow / p.rep, r = orow % p.rep;
        base = p.rec + ((size_t)row * p.nsplit * p.rep + r) * (D + 2);
        stride = (int64_t)p.rep * (D + 2);
    } else {
        base = p.rec + (size_t)orow * (D + 2);
        stride = p.stride_s;
    }
    const float poison = (p.status && *p.status) ? __int_as_float(0x7fc00000) : 0.f;
    constexpr int kPer = kMaxD / 32;                  // channels per lane
    float m = -INFINITY, l = 0.f, o[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) o[i] = 0.f;
    const int s_lo = p.segs > 1 ? (int)blockIdx.y * p.per_seg : 0;
    const int s_hi = p.segs > 1 ? min(p.parts, s_lo + p.per_seg) : p.parts;
    const size_t out_row = p.segs > 1 ? (size_t)blockIdx.y * gridDim.x + orow : (size_t)orow;
    // kBatch records at a time: all their loads are issued before the first is merged (the merge
    // itself is a serial recurrence, and one load round trip per record made this kernel
    // latency-bound); the order of the merge is unchanged.
    constexpr int kBatch = 4;
    for (int s0 = s_lo + warp; s0 < s_hi; s0 += 8 * kBatch) {
        float ms[kBatch], ls[kBatch], v[kBatch][kPer];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int s = s0 + 8 * b;
            const bool live = s < s_hi;
            const float* rec = base + (live ? s : s0) * stride;
            ms[b] = live ? rec[0] : -INFINITY;
            ls[b] = rec[1];
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const int d = lane + 32 * i;
                v[b][i] = d < D ? rec[2 + d] : 0.f;
            }
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            if (!(ms[b] > -INFINITY)) continue;          // empty slice (warp-uniform)
            const float mn = fmaxf(m, ms[b]);
            const float a = expf(m - mn), bb = expf(ms[b] - mn);   // a = 0 while m = -inf
            l = l * a + ls[b] * bb;
#pragma unroll
            for (int i = 0; i < kPer; ++i) o[i] = o[i] * a + v[b][i] * bb;
            m = mn;
        }
    }
    if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
    for (int i = 0; i < kPer; ++i) {
        const int d = lane + 32 * i;
        if (d < D) sm_o[warp][d] = o[i];
    }
    __syncthreads();
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, wgt[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        wgt[w] = (sm_m[w] > -INFINITY) ? expf(sm_m[w] - M) : 0.f;
        L += sm_l[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < D; d += kCombineThreads) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) a += sm_o[w][d] * wgt[w];
        a += poison;
        if (p.normalise) p.out[out_row * D + d] = a / fmaxf(L, 1e-20f);
        else p.out[out_row * (D + 2) + 2 + d] = a;
    }
    if (!p.normalise && threadIdx.x == 0) {
        p.out[out_row * (D + 2) + 0] = M;
        p.out[out_row * (D + 2) + 1] = L;
    }
}

// ---- split plan -------------------------------------------------------------------------------
struct Plan {
    int nsplit, bps;      // work items per cache row, blocks per item
    int bps2, nbig;       // tensor-core kernel: the first nbig items of a row take bps blocks, the rest bps2
    int parts;            // records per cache row and query head (the tensor-core kernel writes one per consumer warp)
    int segs;             // > 1: the merge runs in two levels, `segs` partial merges per output row first
    bool mma;             // tensor-core kernel (persistent, work items of `bps` blocks)
    int grid;
};

constexpr size_t kHeaderBytes = 256;   // work counter + status word in front of the records
constexpr int kCombineDirect = 256;    // up to this many records per output row one CTA merges them all
constexpr int kCombineSegs = 32;       // above it: this many CTAs per row merge a slice each, then one merges those

static bool mma_shape_ok(int D, int group, int rep) {
    return (D == 64 || D == 128) && (group == 16 || group == 32 || group == 64) && D % group == 0 && rep <= 8;
}

static bool force_generic() {
    const char* e = getenv("GKV_DECODE_KERNEL");
    return e && strcmp(e, "generic") == 0;
}

static Plan make_plan(int rows, int nb, int D, int group, int rep, bool allow_mma) {
    Plan pl;
    pl.mma = allow_mma && mma_shape_ok(D, group, rep) && !force_generic();
    if (pl.mma) {
        pl.grid = mma::kCtasPerSM * kNumSM;
        const long total = (long)rows * nb;
        const int nw = mma::kConsumerWarps;
        int chunk = (int)(total / ((long)pl.grid * 6));      // ~6 items per CTA; larger items measured faster than finer balance
        if (chunk < nw) chunk = nw;
        if (chunk > 32) chunk = 32;                      // the producer's metadata table holds 32 blocks
        if (const char* e = getenv("GKV_DECODE_CHUNK")) {      // tuning knob: blocks per work item
            const int v = atoi(e);
            if (v >= 1 && v <= 32) chunk = v;
        }
        // The last part of every row's (rung-sorted) list goes out in half-size items: items are
        // handed out chunk-major, so these are the last items of the grid, and the spread of the
        // CTAs' finishing times is about one item.
        int tail_pct = 0;
        if (const char* e = getenv("GKV_DECODE_TAIL")) {       // tuning knob: percent of a row in half-size items
            const int v = atoi(e);
            if (v >= 0 && v <= 100) tail_pct = v;
        }
        int chunk2 = chunk / 2 < nw ? nw : chunk / 2;
        if (chunk2 > chunk) chunk2 = chunk;
        int nbig = nb > 0 ? (int)(((long)nb * (100 - tail_pct) / 100) / chunk) : 0;
        if (nb / chunk < 4) nbig = (nb + chunk - 1) / chunk;   // short rows: uniform items
        const int rest = nb - nbig * chunk > 0 ? nb - nbig * chunk : 0;
        pl.bps = chunk; pl.bps2 = chunk2; pl.nbig = nbig;
        pl.nsplit = nb > 0 ? nbig + (rest + chunk2 - 1) / chunk2 : 1;
        pl.parts = pl.nsplit * mma::kConsumerWarps;
        pl.segs = pl.parts > kCombineDirect ? (pl.parts / 64 < kCombineSegs ? pl.parts / 64 : kCombineSegs) : 1;
        const long items = (long)rows * pl.nsplit;
        if (items < pl.grid) pl.grid = (int)(items > 0 ? items : 1);
        return pl;
    }
    // generic kernel: enough slices for ~4 CTAs per SM
    int nsplit = (kNumSM * 4 + rows - 1) / rows;
    if (nsplit > nb) nsplit = nb;
    if (nsplit < 1) nsplit = 1;
    pl.bps = nb > 0 ? (nb + nsplit - 1) / nsplit : 1;
    pl.nsplit = nb > 0 ? (nb + pl.bps - 1) / pl.bps : 1;
    pl.parts = pl.nsplit;
    pl.segs = 1;
    pl.grid = 0;
    pl.bps2 = pl.bps; pl.nbig = pl.nsplit;
    return pl;
}

static size_t records_bytes(int B, int Hq, const Plan& pl, int D) {
    return (size_t)B * Hq * ((size_t)pl.parts + (pl.segs > 1 ? pl.segs : 0)) * (D + 2) * sizeof(float);
}

// the tensor-core kernel's rung-sorted block lists: one 16-byte entry per block of every metadata row
static size_t perm_bytes(int rows, int nb) { return (((size_t)rows * nb * sizeof(uint4)) + 255) & ~(size_t)255; }

// Upper bound over both kernels, so the caller's buffer fits whichever is dispatched.
static size_t workspace_bytes(int B, int Hq, int Hkv, int D, int nb) {
    const int rows = B * Hkv, rep = Hq / (Hkv > 0 ? Hkv : 1);
    size_t need = records_bytes(B, Hq, make_plan(rows, nb, D, 32, rep, false), D);
    const size_t alt = records_bytes(B, Hq, make_plan(rows, nb, 128, 32, 1, true), D);
    if (alt > need) need = alt;
    return ((kHeaderBytes + need + 255) & ~(size_t)255) + perm_bytes(rows, nb);
}

template <int D, int G>
static int launch_mma(const mma::Params& p, int grid, cudaStream_t stream) {
    static bool attr_set = false;
    if (!attr_set) {
        GKV_CUDA_TRY(cudaFuncSetAttribute(mma::decode_mma_kernel<D, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)mma::Cfg<D, G>::SMEM));
        attr_set = true;
    }
    mma::decode_mma_kernel<D, G><<<grid, mma::kThreads, mma::Cfg<D, G>::SMEM, stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

static int decode_impl(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                       const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                       const int32_t* valid, float* out, int normalise, void* workspace,
                       size_t ws_bytes, int B, int Hq, int Hkv, int D, int nb, int block, int group,
                       int64_t stride_bh, int meta_rows, void* stream_) {
    if (block != kP) return GKV_E_BLOCK;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || nb < 0 || group <= 0) return GKV_E_SHAPE;
    if (D <= 0 || D > kMaxD || D % 8 != 0) return GKV_E_SHAPE;
    const int rep = Hq / Hkv, rows = B * Hkv;
    if (rep > 16) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (!q || !out) return GKV_E_NULL;
    if (nb > 0 && (!data || !offs || !klo || !kstep || !vlo || !vstep || !level || !valid)) return GKV_E_NULL;
    const size_t need = workspace_bytes(B, Hq, Hkv, D, nb);
    if (!workspace || ws_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255)) return GKV_E_WORKSPACE;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    const bool scales_aligned = ((reinterpret_cast<uintptr_t>(klo) | reinterpret_cast<uintptr_t>(kstep) |
                                  reinterpret_cast<uintptr_t>(vlo) | reinterpret_cast<uintptr_t>(vstep)) & 15) == 0;
    const Plan pl = make_plan(rows, nb, D, group, rep, scales_aligned && nb > 0);
    int* header = static_cast<int*>(workspace);
    float* records = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kHeaderBytes);

    if (pl.mma) {
        // the block lists sit at the end of the workspace, behind the records of either kernel
        uint4* plan = reinterpret_cast<uint4*>(static_cast<uint8_t*>(workspace) + need - perm_bytes(rows, nb));
        int plan_threads = (nb + 31) & ~31;                     // one block per thread up to the CTA limit
        plan_threads = plan_threads < 32 ? 32 : plan_threads > mma::kPlanMaxThreads ? mma::kPlanMaxThreads : plan_threads;
        mma::plan_kernel<<<meta_rows, plan_threads, 0, stream>>>(level, valid, offs, plan, nb, header, (int)(kHeaderBytes / 4));
        GKV_LAUNCH_CHECK();
        mma::Params mp;
        mp.plan = plan; mp.rows = rows;
        mp.q = q; mp.data = data; mp.offs = offs;
        mp.klo = static_cast<const __half*>(klo); mp.kstep = static_cast<const __half*>(kstep);
        mp.vlo = static_cast<const __half*>(vlo); mp.vstep = static_cast<const __half*>(vstep);
        mp.level = level; mp.valid = valid; mp.part = records; mp.counter = header; mp.status = header + 1;
        mp.B = B; mp.Hq = Hq; mp.Hkv = Hkv; mp.nb = nb; mp.rep = rep; mp.chunk = pl.bps; mp.chunk2 = pl.bps2; mp.nbig = pl.nbig;
        mp.items_per_row = pl.nsplit; mp.items = rows * pl.nsplit; mp.per_row_meta = meta_rows != 1;
        mp.stride_bh = stride_bh;
        int rc;
        if (D == 128 && group == 32) rc = launch_mma<128, 32>(mp, pl.grid, stream);
        else if (D == 128 && group == 16) rc = launch_mma<128, 16>(mp, pl.grid, stream);
        else if (D == 128 && group == 64) rc = launch_mma<128, 64>(mp, pl.grid, stream);
        else if (D == 64 && group == 32) rc = launch_mma<64, 32>(mp, pl.grid, stream);
        else if (D == 64 && group == 16) rc = launch_mma<64, 16>(mp, pl.grid, stream);
        else rc = launch_mma<64, 64>(mp, pl.grid, stream);
        if (rc) return rc;
    } else {
        DecodeParams p;
        p.q = q; p.data = data; p.offs = offs;
        p.klo = static_cast<const __half*>(klo); p.kstep = static_cast<const __half*>(kstep);
        p.vlo = static_cast<const __half*>(vlo); p.vstep = static_cast<const __half*>(vstep);
        p.level = level; p.valid = valid;
        p.part = records;
        p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.D = D; p.nb = nb; p.group = group;
        p.G = (kP + group - 1) / group; p.gv = (D + group - 1) / group; p.rep = rep;
        p.nsplit = pl.nsplit; p.bps = pl.bps; p.per_row_meta = meta_rows != 1; p.stride_bh = stride_bh;
        const size_t smem = decode_generic_smem(rep, D);
        static bool attr_set = false;
        if (!attr_set) {
            GKV_CUDA_TRY(cudaFuncSetAttribute(decode_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)decode_generic_smem(16, kMaxD)));
            attr_set = true;
        }
        decode_generic_kernel<<<dim3(pl.nsplit, rows), kGenThreads, smem, stream>>>(p);
        GKV_LAUNCH_CHECK();
    }

    CombineParams c;
    c.rec = records; c.out = out; c.parts = pl.parts; c.D = D; c.rep = rep; c.nsplit = pl.parts;
    c.stride_s = 0; c.normalise = normalise; c.status = pl.mma ? header + 1 : nullptr;
    c.segs = 1; c.per_seg = 0;
    if (pl.segs > 1) {
        // level 1: (rows, parts, rep, D+2) -> (segs, B*Hq, D+2) behind the records
        float* mid = records + (size_t)B * Hq * pl.parts * (D + 2);
        c.out = mid; c.normalise = 0; c.segs = pl.segs; c.per_seg = (pl.parts + pl.segs - 1) / pl.segs;
        combine_kernel<<<dim3(B * Hq, pl.segs), kCombineThreads, 0, stream>>>(c);
        GKV_LAUNCH_CHECK();
        c.rec = mid; c.out = out; c.parts = pl.segs; c.rep = 0; c.nsplit = 0;
        c.stride_s = (int64_t)B * Hq * (D + 2); c.normalise = normalise; c.segs = 1; c.per_seg = 0;
    }
    combine_kernel<<<B * Hq, kCombineThreads, 0, stream>>>(c);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

}  // namespace gkv

extern "C" {

int gkv_abi_version(void) { return 1; }

int gkv_last_cuda_error(void) { return gkv::g_last_cuda_error; }

const char* gkv_error_string(int code) {
    switch (code) {
        case GKV_OK: return "ok";
        case GKV_E_BLOCK: return "only 64-token blocks are supported";
        case GKV_E_SHAPE: return "unsupported or inconsistent shape";
        case GKV_E_NULL: return "a required pointer is null";
        case GKV_E_WORKSPACE: return "workspace missing, misaligned or too small";
        case GKV_E_CUDA: return "a CUDA call failed (see gkv_last_cuda_error)";
        case GKV_E_ARG: return "an argument is out of range";
        case GKV_E_STATIC_SCRATCH: return "problem too large for the built-in scratch of gkv_mixed_attn_decode_static";
        default: return "unknown error code";
    }
}

size_t gkv_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int nb) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || nb < 0) return 0;
    return gkv::workspace_bytes(B, Hq, Hkv, D, nb);
}

int gkv_decode_kernel_launches(int B, int Hq, int Hkv, int D, int nb, int group) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || D <= 0 || nb < 0 || group <= 0) return 0;
    const gkv::Plan pl = gkv::make_plan(B * Hkv, nb, D, group, Hq / Hkv, nb > 0);
    // tensor-core path: block lists, split kernel, one or two merge levels; generic path: split kernel, merge
    return pl.mma ? 2 + (pl.segs > 1 ? 2 : 1) : 2;
}

int gkv_mixed_attn_decode(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                          const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                          const int32_t* valid, float* out, void* workspace, size_t workspace_bytes,
                          int B, int Hq, int Hkv, int D, int nb, int block, int group,
                          int64_t stride_bh, int meta_rows, void* stream) {
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream);
}

int gkv_mixed_attn_decode_partial(const float* q, const uint8_t* data, const int64_t* offs,
                                  const void* klo, const void* kstep, const void* vlo, const void* vstep,
                                  const int32_t* level, const int32_t* valid, float* partial,
                                  void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D,
                                  int nb, int block, int group, int64_t stride_bh, int meta_rows,
                                  void* stream) {
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, partial, 0, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream);
}

int gkv_combine_partials(const float* partials, float* out, int parts, int rows, int D, void* stream) {
    if (!partials || !out) return GKV_E_NULL;
    if (parts <= 0 || rows <= 0 || D <= 0) return GKV_E_SHAPE;
    gkv::CombineParams c;
    c.rec = partials; c.out = out; c.parts = parts; c.D = D; c.rep = 0; c.nsplit = 0;
    c.stride_s = (int64_t)rows * (D + 2); c.normalise = 1; c.status = nullptr; c.segs = 1; c.per_seg = 0;
    gkv::combine_kernel<<<rows, gkv::kCombineThreads, 0, static_cast<cudaStream_t>(stream)>>>(c);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

// ---- decode without any allocation by anyone ------------------------------------------------------
// Scratch for gkv_mixed_attn_decode_static.  It lives in the library image: every GPU that loads
// the library carries these bytes until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[GKV_STATIC_SCRATCH_BYTES];

int gkv_mixed_attn_decode_static(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                                 const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                                 const int32_t* valid, float* out, int B, int Hq, int Hkv, int D, int nb,
                                 int block, int group, int64_t stride_bh, int meta_rows, void* stream) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || nb < 0 || Hq % Hkv != 0) return GKV_E_SHAPE;
    const size_t need = gkv::workspace_bytes(B, Hq, Hkv, D, nb);
    if (need > (size_t)GKV_STATIC_SCRATCH_BYTES) return GKV_E_STATIC_SCRATCH;
    // `g_static_scratch` is only a host-side handle here; the device address has to be asked for,
    // once per device, with that device current.
    constexpr int kMaxDevices = 64;
    static void* device_ptr[kMaxDevices] = {nullptr};
    int dev = 0;
    GKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return GKV_E_ARG;
    if (!device_ptr[dev]) {
        void* ptr = nullptr;
        GKV_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return GKV_E_CUDA;
        device_ptr[dev] = ptr;
    }
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, device_ptr[dev],
                            (size_t)GKV_STATIC_SCRATCH_BYTES, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows,
                            stream);
}

}  // extern "C"
