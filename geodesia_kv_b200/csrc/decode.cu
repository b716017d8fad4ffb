// Decode attention over the packed cache: planning, the LSE combine and the C ABI.

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
    float2* ml_out;      // optional, final level only: (M, L) of every output row (for the per-block softmax mass)
    // Internal layout written by the tensor-core kernel: a row's used item slots are a prefix of its
    // slots (the rest hold "empty" records), and how many are used follows from the row's rung-class
    // counts — so the merge reads only the records that exist.  Null for other producers.
    const int32_t* plan_tab;
    int chunk, tab_per_row, warps_per_item;
};

// Records of output row `orow` that can be non-empty.
__device__ __forceinline__ int live_parts(const CombineParams& p, int orow) {
    if (!p.plan_tab || p.rep <= 0) return p.parts;
    const int32_t* tab = p.plan_tab + (size_t)(p.tab_per_row ? orow / p.rep : 0) * 8;
    int used = 0;
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        const int ck = k == 4 ? min(p.chunk, mma::kMaxCentroidItemBlocks) : p.chunk;     // as the kernel cuts the runs
        used += (tab[k + 1] - tab[k] + ck - 1) / ck;
    }
    return min(p.parts, used * p.warps_per_item);
}

constexpr int kCombineThreads = 256;

// One CTA per output row.  The records of a row are shared out over the NW warps (record s goes
// to warp s mod NW, whose lanes read it coalesced), each warp keeps a running (m, l, o) of its
// records, and the NW states are merged through shared memory — the same recurrence at both levels.
// NW = 8 normally; 32 for rows with a few hundred records, which one wide CTA merges faster than
// two launches of narrow ones (the single-sequence case, where the call is launch-bound).
// KPER = channels per lane (D <= 32 * KPER): head dims up to 128 take the instantiation with half the
// registers, which lets half as many more CTAs sit on an SM (the kernel is bound by the latency of its few
// loads per warp, i.e. by how many CTAs are resident).
template <int NW, int KPER = kMaxD / 32>
__global__ void __launch_bounds__(NW * 32) combine_kernel(CombineParams p) {
    __shared__ float sm_m[NW], sm_l[NW], sm_o[NW][32 * KPER];
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
    constexpr int kPer = KPER;                        // channels per lane
    float m = -INFINITY, l = 0.f, o[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) o[i] = 0.f;
    const int parts = live_parts(p, orow);
    const int s_lo = p.segs > 1 ? (int)blockIdx.y * p.per_seg : 0;
    const int s_hi = p.segs > 1 ? min(parts, s_lo + p.per_seg) : parts;
    const size_t out_row = p.segs > 1 ? (size_t)blockIdx.y * gridDim.x + orow : (size_t)orow;
    // kBatch records at a time: all their loads are issued before the first is merged (the merge
    // itself is a serial recurrence, and one load round trip per record made this kernel
    // latency-bound); the order of the merge is unchanged.
    constexpr int kBatch = KPER <= 4 ? 8 : 4;         // as many as fit the registers
    for (int s0 = s_lo + warp; s0 < s_hi; s0 += NW * kBatch) {
        float ms[kBatch], ls[kBatch], v[kBatch][kPer];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int s = s0 + NW * b;
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
    for (int w = 0; w < NW; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, wgt[NW];
#pragma unroll
    for (int w = 0; w < NW; ++w) {
        wgt[w] = (sm_m[w] > -INFINITY) ? expf(sm_m[w] - M) : 0.f;
        L += sm_l[w] * wgt[w];
    }
    for (int d = threadIdx.x; d < D; d += NW * 32) {
        float a = 0.f;
#pragma unroll
        for (int w = 0; w < NW; ++w) a += sm_o[w][d] * wgt[w];
        a += poison;
        if (p.normalise) p.out[out_row * D + d] = a / fmaxf(L, 1e-20f);
        else p.out[out_row * (D + 2) + 2 + d] = a;
    }
    if (!p.normalise && threadIdx.x == 0) {
        p.out[out_row * (D + 2) + 0] = M;
        p.out[out_row * (D + 2) + 1] = L;
    }
    if (p.ml_out && p.segs <= 1 && threadIdx.x == 0) p.ml_out[out_row] = make_float2(M, L);
}

// ---- per-block softmax mass -----------------------------------------------------------------------
// mass[row][b] = mean over the row's query heads of (sum over the block's tokens of softmax weight), the
// quantity geodesia_kv/policies.py:1497-1509 obtains from a dense softmax over the keys.  Here it is put
// together from what the decode kernel reported per block half and head — the reference m it was using
// and the sum of exp(s - m) — and the final (M, L) of every head: weight = exp(m - M) * sum / L.
__global__ void block_mass_kernel(const float2* __restrict__ part, const float2* __restrict__ ml,
                                  const int32_t* __restrict__ level, const int32_t* __restrict__ valid,
                                  float* __restrict__ mass, int rows, int nb, int rep, int upb, int per_row_meta) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)rows * nb) return;
    const int row = (int)(i / nb), b = (int)(i % nb);
    const size_t mi = (size_t)(per_row_meta ? row : 0) * nb + b;
    float acc = 0.f;
    if (valid[mi] > 0 && level_ok(level[mi])) {
        for (int h = 0; h < rep; ++h) {
            const float2 f = ml[(size_t)row * rep + h];
            float w = 0.f;
            for (int u = 0; u < upb; ++u) {
                const float2 pr = part[(i * upb + u) * rep + h];
                if (pr.x > -INFINITY) w += expf(pr.x - f.x) * pr.y;
            }
            acc += w / fmaxf(f.y, 1e-20f);
        }
        acc /= (float)rep;
    }
    mass[i] = acc;
}

// ---- final merge of a sequence that is split over several GPUs ------------------------------------
// Every rank holds, per output row, the records of its own slice of the sequence.  This kernel is the
// last merge level of the rank's decode AND the exchange between the ranks: the CTA of an output row
// merges the local records into one (m, l, o), stores it into the inbox of every rank (its own
// included) with plain peer stores, raises the row's sequence number in every inbox (release), waits
// until all `world` records of that sequence number have arrived in its own inbox (acquire, bounded)
// and merges them into the normalised output.  No collective library is involved, and nothing but
// this library's kernels runs in the step.
//
// Inbox of one rank: records [2][world][rows][D+2] floats (indexed by the parity of the sequence
// number: a rank can be at most one call ahead of a peer, so two buffers never collide) followed by
// flags [world][rows] ints.  seq[rows] lives in local memory and counts this row's calls; all ranks
// must make the same calls in the same order.
constexpr int kMaxWorld = 8;
struct ExchangeParams {
    float* inbox[kMaxWorld];
    int* flags[kMaxWorld];
    int* seq;
    int* xstatus;        // sticky error word of the exchange (non-zero: a wait ran out)
    int rank, world, rows;
    unsigned long long wait_ns;   // how long a rank waits for the others' records before it gives up
};

// Process-wide limit of that wait (gkv_set_exchange_wait_ns); one second unless a host says otherwise.
static unsigned long long g_exchange_wait_ns = 1000000000ull;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kCombineThreads) exchange_combine_kernel(CombineParams p, ExchangeParams x) {
    __shared__ float sm_m[8], sm_l[8], sm_o[8][kMaxD];
    __shared__ float xm[kMaxWorld], xl[kMaxWorld];
    __shared__ int s_seq, s_fail;
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
    const bool local_fail = p.status && *p.status;
    constexpr int kPer = kMaxD / 32;
    float m = -INFINITY, l = 0.f, o[kPer];
#pragma unroll
    for (int i = 0; i < kPer; ++i) o[i] = 0.f;
    constexpr int kBatch = 4;
    const int parts = live_parts(p, orow);
    for (int s0 = warp; s0 < parts; s0 += 8 * kBatch) {
        float ms[kBatch], ls[kBatch], v[kBatch][kPer];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int s = s0 + 8 * b;
            const bool live = s < parts;
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
            if (!(ms[b] > -INFINITY)) continue;
            const float mn = fmaxf(m, ms[b]);
            const float a = expf(m - mn), bb = expf(ms[b] - mn);
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
    if (threadIdx.x == 0) { s_seq = x.seq[orow] + 1; s_fail = 0; }
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
    const int seq = s_seq, par = seq & 1;
    // this rank's record of the row goes to every inbox
    const size_t slot = ((size_t)(par * x.world + x.rank) * x.rows + orow) * (D + 2);
    for (int d = threadIdx.x; d < D + 2; d += kCombineThreads) {
        float a;
        if (d == 0) a = M;
        else if (d == 1) a = L;
        else {
            a = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) a += sm_o[w][d - 2] * wgt[w];
        }
        for (int r = 0; r < x.world; ++r) x.inbox[r][slot + d] = a;
    }
    __threadfence_system();                 // every thread's record stores are visible system-wide ...
    __syncthreads();
    // ... before the sequence numbers go out: one relaxed store per destination rank, issued by `world`
    // threads at once (a release store per rank from one thread would serialise a round trip each)
    if (threadIdx.x < x.world) st_relaxed_sys(x.flags[threadIdx.x] + (size_t)x.rank * x.rows + orow, seq);
    if (threadIdx.x == 0) x.seq[orow] = seq;
    // one thread per source rank waits for that rank's record of this call
    if (threadIdx.x < x.world) {
        const int* f = x.flags[x.rank] + (size_t)threadIdx.x * x.rows + orow;
        unsigned long long t0 = 0;
        bool got = false;
        for (unsigned spin = 0;; ++spin) {
            if (ld_acquire_sys(f) - seq >= 0) { got = true; break; }
            if (spin > 16) __nanosleep(64);
            if ((spin & 255u) == 255u) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                else if (now - t0 > x.wait_ns) break;
            }
        }
        if (!got) { s_fail = 1; atomicExch(x.xstatus, 1 + (int)threadIdx.x); }
    }
    __syncthreads();
    const float* mine = x.inbox[x.rank] + (size_t)par * x.world * x.rows * (D + 2);
    if (threadIdx.x < x.world) {
        const float* rec = mine + ((size_t)threadIdx.x * x.rows + orow) * (D + 2);
        xm[threadIdx.x] = __ldcg(rec);
        xl[threadIdx.x] = __ldcg(rec + 1);
    }
    __syncthreads();
    float GM = -INFINITY;
    for (int r = 0; r < x.world; ++r) GM = fmaxf(GM, xm[r]);
    float GL = 0.f, gw[kMaxWorld];
#pragma unroll
    for (int r = 0; r < kMaxWorld; ++r) {
        gw[r] = (r < x.world && xm[r] > -INFINITY) ? expf(xm[r] - GM) : 0.f;
        if (r < x.world) GL += xl[r] * gw[r];
    }
    const float poison = (local_fail || s_fail) ? __int_as_float(0x7fc00000) : 0.f;
    for (int d = threadIdx.x; d < D; d += kCombineThreads) {
        float a = 0.f;
        for (int r = 0; r < x.world; ++r) a += __ldcg(mine + ((size_t)r * x.rows + orow) * (D + 2) + 2 + d) * gw[r];
        p.out[(size_t)orow * D + d] = a / fmaxf(GL, 1e-20f) + poison;
    }
}

// ---- split plan -------------------------------------------------------------------------------
struct Plan {
    int nsplit, bps;      // work items (tensor-core kernel: item slots) per cache row, blocks per item
    int parts;            // records per cache row and query head (the tensor-core kernel writes one per consumer warp)
    int segs;             // > 1: the merge runs in two levels, `segs` partial merges per output row first
    bool mma;             // tensor-core kernel (persistent, work items of `bps` blocks)
    bool wide = false;    // one merge level by a CTA of 32 warps (a few hundred records per row)
    int grid;
};

constexpr size_t kHeaderBytes = 256;   // work counter + status word in front of the records
constexpr int kAutoItemBlocks = 64;     // largest work item the planner picks by itself
constexpr int kCombineDirect = 256;    // up to this many records per output row one CTA merges them all
constexpr int kCombineWide = 256;      // up to this many, one CTA of 32 warps would (measured slower than two levels on the
                                       // single-sequence case, 34.8 against 28.7 us per call: not used, same as kCombineDirect)
constexpr int kCombineSegs = 32;       // above it: this many CTAs per row merge a slice each, then one merges those

static bool mma_shape_ok(int D, int group, int rep) {
    return (D == 64 || D == 128) && (group == 16 || group == 32 || group == 64) && D % group == 0 && rep <= 8;
}

// Process-wide kernel choice (gkv_set_decode_kernel): 0 = by shape, 1 = always the CUDA-core kernel.
static int g_decode_kernel = 0;
static bool force_generic() { return g_decode_kernel == 1; }
// Process-wide override of the tensor-core kernel's work-item size (gkv_set_decode_item_blocks): 0 = by problem size.
static int g_item_blocks = 0;

// Per-device facts and one-time set-up, keyed by the CUDA device ordinal (a process may drive
// several GPUs; function attributes and the SM count belong to the device, not the process).
constexpr int kMaxDevices = 64;
static int g_sm_count[kMaxDevices] = {0};

static int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
    return dev;
}

// Multiprocessors of the current device (148 on B200); `fallback` when no device answers, so that
// the pure-host size queries still work on a machine without a GPU.
static int sm_count(int fallback = kNumSM) {
    const int dev = current_device();
    if (dev < 0) return fallback;
    if (g_sm_count[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            return fallback;
        }
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

static Plan make_plan(int rows, int nb, int D, int group, int rep, bool allow_mma) {
    Plan pl;
    const int sms = sm_count();
    pl.mma = allow_mma && mma_shape_ok(D, group, rep) && !force_generic();
    if (pl.mma) {
        pl.grid = mma::kCtasPerSM * sms;
        const long total = (long)rows * nb;
        // One item per CTA where the problem allows it, never more than 64 blocks per item: large items
        // measured faster than fine balance at every size (a 1M-token row cut in 2, 4, 8: items of 48-64
        // blocks beat items of 9-37 by up to 30 %), small ones only pay off when there are fewer blocks
        // than would keep every SM busy (the single-sequence call).
        int chunk = (int)((total + pl.grid - 1) / pl.grid);
        if (chunk < mma::kMinItemBlocks) chunk = mma::kMinItemBlocks;
        if (chunk > kAutoItemBlocks) chunk = kAutoItemBlocks;            // larger items (up to mma::kMaxItemBlocks, by
                                                                         // gkv_set_decode_item_blocks) measured no faster
        if (g_item_blocks > 0) chunk = g_item_blocks;
        // Every rung's run of a row's sorted list is cut into items of `chunk` blocks; whatever the
        // mix of rungs, ceil(nb / chunk) + 4 slots hold them all (five runs, each with one short item
        // at most).  Slots a row does not need stay empty.
        pl.bps = chunk;
        const int cmin = chunk < mma::kMaxCentroidItemBlocks ? chunk : mma::kMaxCentroidItemBlocks;
        pl.nsplit = (nb + cmin - 1) / cmin + 4;
        pl.parts = pl.nsplit * mma::kConsumerWarps;
        pl.wide = pl.parts > kCombineDirect && pl.parts <= kCombineWide;
        pl.segs = pl.parts > kCombineWide ? (pl.parts / 64 < kCombineSegs ? pl.parts / 64 : kCombineSegs) : 1;
        return pl;
    }
    // generic kernel: enough slices for ~4 CTAs per SM
    int nsplit = (sms * 4 + rows - 1) / rows;
    if (nsplit > nb) nsplit = nb;
    if (nsplit < 1) nsplit = 1;
    pl.bps = nb > 0 ? (nb + nsplit - 1) / nsplit : 1;
    pl.nsplit = nb > 0 ? (nb + pl.bps - 1) / pl.bps : 1;
    pl.parts = pl.nsplit;
    pl.segs = 1;
    pl.grid = 0;
    return pl;
}

static size_t records_bytes(int B, int Hq, const Plan& pl, int D) {
    return (size_t)B * Hq * ((size_t)pl.parts + (pl.segs > 1 ? pl.segs : 0)) * (D + 2) * sizeof(float);
}

// the tensor-core kernel's rung-sorted block lists: one 16-byte entry per block of every metadata row,
// followed by the rows' tables of where each rung starts in its list
static size_t perm_entries_bytes(int rows, int nb) { return (((size_t)rows * nb * sizeof(uint4)) + 255) & ~(size_t)255; }
static size_t perm_bytes(int rows, int nb) {
    return perm_entries_bytes(rows, nb) + ((((size_t)rows * mma::kPlanTabInts * sizeof(int32_t)) + 255) & ~(size_t)255);
}

// Upper bound over both kernels, so the caller's buffer fits whichever is dispatched.
static size_t workspace_bytes(int B, int Hq, int Hkv, int D, int nb) {
    const int rows = B * Hkv, rep = Hq / (Hkv > 0 ? Hkv : 1);
    size_t need = records_bytes(B, Hq, make_plan(rows, nb, D, 32, rep, false), D);
    const size_t alt = records_bytes(B, Hq, make_plan(rows, nb, 128, 32, 1, true), D);
    if (alt > need) need = alt;
    return ((kHeaderBytes + need + 255) & ~(size_t)255) + perm_bytes(rows, nb);
}

// A kernel that needs more than 48 KB of dynamic shared memory has to be opted in once per device.
// extra scratch of a decode that also reports the per-block softmax mass: the kernel's partials and the heads' (M, L)
static size_t mass_bytes(int B, int Hq, int Hkv, int nb, int group) {
    const size_t rows = (size_t)B * Hkv, rep = (size_t)(Hq / (Hkv > 0 ? Hkv : 1));
    const size_t upb = group > 0 && group <= kP ? (size_t)(kP / group) : 1;
    return ((rows * nb * upb * rep + (size_t)B * Hq) * sizeof(float2) + 255) & ~(size_t)255;
}

template <typename Kernel>
static int opt_in_smem(Kernel kernel, unsigned char (&done)[kMaxDevices], size_t bytes) {
    const int dev = current_device();
    if (dev < 0) return GKV_E_CUDA;
    if (!done[dev]) {
        GKV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        done[dev] = 1;
    }
    return GKV_OK;
}

// ---- tensor maps of the cache bytes (tiled, swizzled bulk copies) -------------------------------------
// The encoder lives in the driver; it is looked up once through the runtime, so the library links
// nothing but the runtime.
typedef CUresult (*TensorMapEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                      const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                      CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static TensorMapEncodeFn tensor_map_encoder() {
    static TensorMapEncodeFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TensorMapEncodeFn>(ptr);
        else
            cudaGetLastError();
        tried = true;
    }
    return fn;
}

// The cache as a matrix of w-byte rows, a block as a box of `rows` of them.
static bool encode_rows(CUtensorMap* map, const uint8_t* data, size_t total_bytes, int w, int rows) {
    TensorMapEncodeFn enc = tensor_map_encoder();
    if (!enc || w < 32 || rows > 256 || total_bytes / (size_t)w == 0) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)w, (cuuint64_t)(total_bytes / (size_t)w)};
    const cuuint64_t strides[1] = {(cuuint64_t)w};
    const cuuint32_t box[2] = {(cuuint32_t)w, (cuuint32_t)rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = w == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : w == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                                                                                   : CU_TENSOR_MAP_SWIZZLE_32B;
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(data), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, int G>
static void make_tensor_maps(mma::TensorMaps& tm, const uint8_t* data, size_t total_bytes) {
    memset(&tm, 0, sizeof(tm));
    if (reinterpret_cast<uintptr_t>(data) & 15) return;             // the copy engine wants a 16-byte aligned base
    bool ok = true;
    // rows per block = both halves of the block (2 x 64 token rows) in tile rows of w bytes
    { using L = mma::Lay<D, G, 16>; ok = ok && encode_rows(&tm.m[0], data, total_bytes, L::W, 2 * kP * L::RB / L::W); }
    { using L = mma::Lay<D, G, 8>;  ok = ok && encode_rows(&tm.m[1], data, total_bytes, L::W, 2 * kP * L::RB / L::W); }
    if (mma::Lay<D, G, 4>::TILED) {
        using L = mma::Lay<D, G, 4>;
        ok = ok && encode_rows(&tm.m[2], data, total_bytes, L::W, 2 * kP * L::RB / L::W);
    }
    tm.usable = ok ? 1 : 0;
}

template <int D, int G, bool DUP, bool MASS>
static int launch_mma3(const mma::Params& p, const mma::TensorMaps& tm, int grid, cudaStream_t stream) {
    static unsigned char done[kMaxDevices] = {0};
    if (const int rc = opt_in_smem(mma::decode_mma_kernel<D, G, DUP, MASS>, done, mma::Cfg<D, G>::SMEM)) return rc;
    mma::decode_mma_kernel<D, G, DUP, MASS><<<grid, mma::kThreads, mma::Cfg<D, G>::SMEM, stream>>>(p, tm);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

template <int D, int G, bool DUP>
static int launch_mma2(const mma::Params& p, const mma::TensorMaps& tm, int grid, cudaStream_t stream) {
    return p.mass_part ? launch_mma3<D, G, DUP, true>(p, tm, grid, stream) : launch_mma3<D, G, DUP, false>(p, tm, grid, stream);
}

// up to four query heads per cache row: the (hi, lo) halves of a head share one MMA
template <int D, int G>
static int launch_mma(const mma::Params& p, size_t total_bytes, int grid, cudaStream_t stream) {
    mma::TensorMaps tm;
    make_tensor_maps<D, G>(tm, p.data, total_bytes);
    return p.rep <= 4 ? launch_mma2<D, G, true>(p, tm, grid, stream) : launch_mma2<D, G, false>(p, tm, grid, stream);
}

static int launch_plan(const int32_t* level, const int32_t* valid, const int64_t* offs, uint4* plan, int meta_rows,
                       int nb, int* header, cudaStream_t stream) {
    int plan_threads = (nb + 31) & ~31;                     // one block per thread up to the CTA limit
    plan_threads = plan_threads < 32 ? 32 : plan_threads > mma::kPlanMaxThreads ? mma::kPlanMaxThreads : plan_threads;
    int32_t* tab = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(plan) + perm_entries_bytes(meta_rows, nb));
    mma::plan_kernel<<<meta_rows, plan_threads, 0, stream>>>(level, valid, offs, plan, tab, nb, header,
                                                            header ? (int)(kHeaderBytes / 4) : 0);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

static int decode_impl(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                       const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                       const int32_t* valid, float* out, int normalise, const void* plan_in, void* workspace,
                       size_t ws_bytes, int B, int Hq, int Hkv, int D, int nb, int block, int group,
                       int64_t stride_bh, int meta_rows, void* stream_, const ExchangeParams* xch = nullptr,
                       float* mass_out = nullptr, size_t pool_bytes = 0) {
    const bool paged = pool_bytes != 0;        // `data` is a block pool with the scale planes behind each block
    if (block != kP) return GKV_E_BLOCK;
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || nb < 0 || group <= 0) return GKV_E_SHAPE;
    if (D <= 0 || D > kMaxD || D % 8 != 0) return GKV_E_SHAPE;
    const int rep = Hq / Hkv, rows = B * Hkv;
    if (rep > 16) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (!q || !out) return GKV_E_NULL;
    if (nb > 0 && (!data || !offs || !level || !valid)) return GKV_E_NULL;
    if (nb > 0 && !paged && (!klo || !kstep || !vlo || !vstep)) return GKV_E_NULL;
    const size_t need = workspace_bytes(B, Hq, Hkv, D, nb);
    const size_t need_all = need + (mass_out ? mass_bytes(B, Hq, Hkv, nb, group) : 0);
    if (!workspace || ws_bytes < need_all || (reinterpret_cast<uintptr_t>(workspace) & 255)) return GKV_E_WORKSPACE;
    if (plan_in && (reinterpret_cast<uintptr_t>(plan_in) & 15)) return GKV_E_ARG;
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);

    const bool scales_aligned = paged ? (reinterpret_cast<uintptr_t>(data) & 15) == 0
                                      : ((reinterpret_cast<uintptr_t>(klo) | reinterpret_cast<uintptr_t>(kstep) |
                                          reinterpret_cast<uintptr_t>(vlo) | reinterpret_cast<uintptr_t>(vstep)) & 15) == 0;
    const Plan pl = make_plan(rows, nb, D, group, rep, scales_aligned && nb > 0);
    int* header = static_cast<int*>(workspace);
    float* records = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + kHeaderBytes);

    if ((mass_out || paged) && !pl.mma) return GKV_E_SHAPE;  // the by-product and the pool form exist in the tensor-core kernel only
    float2* mass_part = mass_out ? reinterpret_cast<float2*>(static_cast<uint8_t*>(workspace) + need) : nullptr;
    float2* mass_ml = mass_out ? mass_part + (size_t)rows * nb * (kP / group) * rep : nullptr;
    const int32_t* combine_tab = nullptr;
    if (pl.mma) {
        const uint4* plan = static_cast<const uint4*>(plan_in);
        if (plan) {
            // the caller keeps the block lists (they change only with level/valid/offs): only the
            // work counter and the status word have to start at zero
            GKV_CUDA_TRY(cudaMemsetAsync(header, 0, kHeaderBytes, stream));
        } else {
            // the block lists sit at the end of the workspace, behind the records of either kernel
            uint4* mine = reinterpret_cast<uint4*>(static_cast<uint8_t*>(workspace) + need - perm_bytes(meta_rows, nb));
            if (const int rc = launch_plan(level, valid, offs, mine, meta_rows, nb, header, stream)) return rc;
            plan = mine;
        }
        mma::Params mp;
        mp.plan = plan; mp.rows = rows;
        mp.plan_tab = reinterpret_cast<const int32_t*>(reinterpret_cast<const uint8_t*>(plan) + perm_entries_bytes(meta_rows, nb));
        combine_tab = mp.plan_tab;
        mp.q = q; mp.data = data; mp.offs = offs;
        mp.klo = static_cast<const __half*>(klo); mp.kstep = static_cast<const __half*>(kstep);
        mp.vlo = static_cast<const __half*>(vlo); mp.vstep = static_cast<const __half*>(vstep);
        mp.level = level; mp.valid = valid; mp.part = records; mp.counter = header; mp.status = header + 1;
        mp.mass_part = mass_part;
        mp.B = B; mp.Hq = Hq; mp.Hkv = Hkv; mp.nb = nb; mp.rep = rep; mp.chunk = pl.bps;
        mp.items_per_row = pl.nsplit; mp.items = rows * pl.nsplit; mp.per_row_meta = meta_rows != 1;
        mp.stride_bh = paged ? 0 : stride_bh;
        mp.paged = paged ? 1 : 0;
        int rc;
        const size_t total = paged ? pool_bytes : (size_t)rows * (size_t)stride_bh;   // bytes the tensor maps span
        if (D == 128 && group == 32) rc = launch_mma<128, 32>(mp, total, pl.grid, stream);
#ifdef GKV_FAST_BUILD      // development builds: only the main shape is instantiated
        else rc = GKV_E_SHAPE;
#else
        else if (D == 128 && group == 16) rc = launch_mma<128, 16>(mp, total, pl.grid, stream);
        else if (D == 128 && group == 64) rc = launch_mma<128, 64>(mp, total, pl.grid, stream);
        else if (D == 64 && group == 32) rc = launch_mma<64, 32>(mp, total, pl.grid, stream);
        else if (D == 64 && group == 16) rc = launch_mma<64, 16>(mp, total, pl.grid, stream);
        else rc = launch_mma<64, 64>(mp, total, pl.grid, stream);
#endif
        if (rc) return rc;
    } else {
        GKV_CUDA_TRY(cudaMemsetAsync(header, 0, kHeaderBytes, stream));      // status word reads "ok"
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
        static unsigned char done[kMaxDevices] = {0};
        if (const int rc = opt_in_smem(decode_generic_kernel, done, decode_generic_smem(16, kMaxD))) return rc;
        decode_generic_kernel<<<dim3(pl.nsplit, rows), kGenThreads, smem, stream>>>(p);
        GKV_LAUNCH_CHECK();
    }

    CombineParams c;
    c.rec = records; c.out = out; c.parts = pl.parts; c.D = D; c.rep = rep; c.nsplit = pl.parts;
    c.stride_s = 0; c.normalise = normalise; c.status = pl.mma ? header + 1 : nullptr;
    c.segs = 1; c.per_seg = 0; c.ml_out = nullptr;
    c.plan_tab = nullptr; c.chunk = 1; c.tab_per_row = 0; c.warps_per_item = 1;
    if (pl.mma) {
        c.plan_tab = combine_tab; c.chunk = pl.bps; c.tab_per_row = meta_rows != 1; c.warps_per_item = mma::kConsumerWarps;
    }
    if (pl.segs > 1) {
        // level 1: (rows, parts, rep, D+2) -> (segs, B*Hq, D+2) behind the records
        float* mid = records + (size_t)B * Hq * pl.parts * (D + 2);
        c.out = mid; c.normalise = 0; c.segs = pl.segs; c.per_seg = (pl.parts + pl.segs - 1) / pl.segs;
        if (D <= 128) combine_kernel<8, 4><<<dim3(B * Hq, pl.segs), kCombineThreads, 0, stream>>>(c);
        else combine_kernel<8><<<dim3(B * Hq, pl.segs), kCombineThreads, 0, stream>>>(c);
        GKV_LAUNCH_CHECK();
        c.rec = mid; c.out = out; c.parts = pl.segs; c.rep = 0; c.nsplit = 0; c.plan_tab = nullptr;
        c.stride_s = (int64_t)B * Hq * (D + 2); c.normalise = normalise; c.segs = 1; c.per_seg = 0;
    }
    c.ml_out = mass_ml;
    if (xch) exchange_combine_kernel<<<B * Hq, kCombineThreads, 0, stream>>>(c, *xch);
    else if (pl.wide && pl.segs <= 1) combine_kernel<32><<<B * Hq, 1024, 0, stream>>>(c);
    else if (D <= 128) combine_kernel<8, 4><<<B * Hq, kCombineThreads, 0, stream>>>(c);
    else combine_kernel<8><<<B * Hq, kCombineThreads, 0, stream>>>(c);
    GKV_LAUNCH_CHECK();
    if (mass_out) {
        const size_t n = (size_t)rows * nb;
        block_mass_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(mass_part, mass_ml, level, valid, mass_out, rows, nb,
                                                                       rep, kP / group, meta_rows != 1);
        GKV_LAUNCH_CHECK();
    }
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

int gkv_decode_launch_count(int B, int Hq, int Hkv, int D, int nb, int group, int planned) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || D <= 0 || nb < 0 || group <= 0) return 0;
    const gkv::Plan pl = gkv::make_plan(B * Hkv, nb, D, group, Hq / Hkv, nb > 0);
    // tensor-core path: block lists (unless the caller keeps them), split kernel, one or two merge
    // levels; generic path: split kernel, merge
    return pl.mma ? (planned ? 1 : 2) + (pl.segs > 1 ? 2 : 1) : 2;
}

int gkv_decode_kernel_launches(int B, int Hq, int Hkv, int D, int nb, int group) {
    return gkv_decode_launch_count(B, Hq, Hkv, D, nb, group, 0);
}

int gkv_set_decode_kernel(int which) {
    if (which != 0 && which != 1) return GKV_E_ARG;
    gkv::g_decode_kernel = which;
    return GKV_OK;
}

int gkv_set_decode_item_blocks(int blocks) {
    if (blocks != 0 && (blocks < 1 || blocks > gkv::mma::kMaxItemBlocks)) return GKV_E_ARG;
    gkv::g_item_blocks = blocks;
    return GKV_OK;
}

size_t gkv_decode_plan_bytes(int meta_rows, int nb) {
    if (meta_rows <= 0 || nb < 0) return 0;
    return gkv::perm_bytes(meta_rows, nb > 0 ? nb : 1);
}

int gkv_decode_build_plan(const int64_t* offs, const int32_t* level, const int32_t* valid, void* plan,
                          int meta_rows, int nb, void* stream) {
    if (meta_rows <= 0 || nb < 0) return GKV_E_SHAPE;
    if (nb == 0) return GKV_OK;
    if (!offs || !level || !valid || !plan) return GKV_E_NULL;
    if (reinterpret_cast<uintptr_t>(plan) & 15) return GKV_E_ARG;
    return gkv::launch_plan(level, valid, offs, static_cast<uint4*>(plan), meta_rows, nb, nullptr,
                            static_cast<cudaStream_t>(stream));
}

int gkv_decode_status(const void* workspace, int* status_host, void* stream) {
    if (!workspace || !status_host) return GKV_E_NULL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int word = 0;
    GKV_CUDA_TRY(cudaMemcpyAsync(&word, static_cast<const int*>(workspace) + 1, sizeof(int), cudaMemcpyDeviceToHost, st));
    GKV_CUDA_TRY(cudaStreamSynchronize(st));
    *status_host = word;
    return GKV_OK;
}

int gkv_mixed_attn_decode(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                          const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                          const int32_t* valid, float* out, void* workspace, size_t workspace_bytes,
                          int B, int Hq, int Hkv, int D, int nb, int block, int group,
                          int64_t stride_bh, int meta_rows, void* stream) {
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, nullptr, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream);
}

int gkv_mixed_attn_decode_planned(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                                  const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                                  const int32_t* valid, float* out, const void* plan, int partial,
                                  void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D,
                                  int nb, int block, int group, int64_t stride_bh, int meta_rows,
                                  void* stream) {
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, partial ? 0 : 1, plan,
                            workspace, workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows,
                            stream);
}

int gkv_mixed_attn_decode_partial(const float* q, const uint8_t* data, const int64_t* offs,
                                  const void* klo, const void* kstep, const void* vlo, const void* vstep,
                                  const int32_t* level, const int32_t* valid, float* partial,
                                  void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D,
                                  int nb, int block, int group, int64_t stride_bh, int meta_rows,
                                  void* stream) {
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, partial, 0, nullptr, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream);
}

size_t gkv_decode_mass_workspace_bytes(int B, int Hq, int Hkv, int D, int nb, int group) {
    if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0 || nb < 0 || group <= 0) return 0;
    return gkv::workspace_bytes(B, Hq, Hkv, D, nb) + gkv::mass_bytes(B, Hq, Hkv, nb, group);
}

int gkv_mixed_attn_decode_mass(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                               const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                               const int32_t* valid, float* out, float* mass, const void* plan, void* workspace,
                               size_t workspace_bytes, int B, int Hq, int Hkv, int D, int nb, int block,
                               int group, int64_t stride_bh, int meta_rows, void* stream) {
    if (!mass) return GKV_E_NULL;
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, plan, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream, nullptr,
                            mass);
}

int gkv_paged_attn_decode(const float* q, const uint8_t* pool, size_t pool_bytes, const int64_t* offs,
                          const int32_t* level, const int32_t* valid, float* out, float* mass_out, const void* plan,
                          void* workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D, int nb, int block,
                          int group, void* stream) {
    if (pool_bytes == 0 && nb > 0) return GKV_E_ARG;
    return gkv::decode_impl(q, pool, offs, nullptr, nullptr, nullptr, nullptr, level, valid, out, 1, plan, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, 0, B * Hkv, stream, nullptr, mass_out,
                            pool_bytes ? pool_bytes : 1);
}

int gkv_set_exchange_wait_ns(unsigned long long ns) {
    if (ns == 0) return GKV_E_ARG;
    gkv::g_exchange_wait_ns = ns;
    return GKV_OK;
}

size_t gkv_exchange_inbox_bytes(int world, int rows, int D) {
    if (world <= 0 || world > gkv::kMaxWorld || rows <= 0 || D <= 0) return 0;
    const size_t rec = (size_t)2 * world * rows * (D + 2) * sizeof(float);
    const size_t flags = (size_t)world * rows * sizeof(int);
    return ((rec + 255) & ~(size_t)255) + ((flags + 255) & ~(size_t)255);
}

int gkv_mixed_attn_decode_exchange(const float* q, const uint8_t* data, const int64_t* offs, const void* klo,
                                   const void* kstep, const void* vlo, const void* vstep, const int32_t* level,
                                   const int32_t* valid, float* out, const void* plan, void* workspace,
                                   size_t workspace_bytes, int B, int Hq, int Hkv, int D, int nb, int block,
                                   int group, int64_t stride_bh, int meta_rows, void* const* inboxes, int rank,
                                   int world, int* seq, int* xstatus, void* stream) {
    if (!inboxes || !seq || !xstatus) return GKV_E_NULL;
    if (world <= 0 || world > gkv::kMaxWorld || rank < 0 || rank >= world) return GKV_E_ARG;
    if (B <= 0 || Hq <= 0 || D <= 0) return GKV_E_SHAPE;
    gkv::ExchangeParams x;
    const int rows = B * Hq;
    const size_t rec = (((size_t)2 * world * rows * (D + 2) * sizeof(float)) + 255) & ~(size_t)255;
    for (int r = 0; r < gkv::kMaxWorld; ++r) {
        if (r < world && !inboxes[r]) return GKV_E_NULL;
        x.inbox[r] = r < world ? static_cast<float*>(inboxes[r]) : nullptr;
        x.flags[r] = r < world ? reinterpret_cast<int*>(static_cast<uint8_t*>(inboxes[r]) + rec) : nullptr;
    }
    x.seq = seq; x.xstatus = xstatus; x.rank = rank; x.world = world; x.rows = rows;
    x.wait_ns = gkv::g_exchange_wait_ns;
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, plan, workspace,
                            workspace_bytes, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows, stream, &x);
}

int gkv_combine_partials(const float* partials, float* out, int parts, int rows, int D, void* stream) {
    if (!partials || !out) return GKV_E_NULL;
    if (parts <= 0 || rows <= 0 || D <= 0) return GKV_E_SHAPE;
    gkv::CombineParams c;
    c.rec = partials; c.out = out; c.parts = parts; c.D = D; c.rep = 0; c.nsplit = 0;
    c.stride_s = (int64_t)rows * (D + 2); c.normalise = 1; c.status = nullptr; c.segs = 1; c.per_seg = 0; c.ml_out = nullptr;
    c.plan_tab = nullptr; c.chunk = 1; c.tab_per_row = 0; c.warps_per_item = 1;
    if (D <= 128) gkv::combine_kernel<8, 4><<<rows, gkv::kCombineThreads, 0, static_cast<cudaStream_t>(stream)>>>(c);
    else gkv::combine_kernel<8><<<rows, gkv::kCombineThreads, 0, static_cast<cudaStream_t>(stream)>>>(c);
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
    static void* device_ptr[gkv::kMaxDevices] = {nullptr};
    int dev = 0;
    GKV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= gkv::kMaxDevices) return GKV_E_ARG;
    if (!device_ptr[dev]) {
        void* ptr = nullptr;
        GKV_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return GKV_E_CUDA;
        device_ptr[dev] = ptr;
    }
    return gkv::decode_impl(q, data, offs, klo, kstep, vlo, vstep, level, valid, out, 1, nullptr, device_ptr[dev],
                            (size_t)GKV_STATIC_SCRATCH_BYTES, B, Hq, Hkv, D, nb, block, group, stride_bh, meta_rows,
                            stream);
}

}  // extern "C"
