// Tensor-core split decode kernel for the packed bit-ladder cache (sm_100a).
//
// Why tensor cores at all: at HBM speed the 16k-token mix delivers ~7.8e12 codes/s per GPU.
// With a GQA group of 4-8 query heads every code needs 4-8 FMAs plus its unpack, which is
// above the FP32 issue rate of the chip (the CUDA-core kernel in decode_generic.cuh measures
// ~3 % of HBM bandwidth).  The group's QK^T and PV products are therefore issued as
// m16n8k16 MMAs straight from registers; the bytes never make a second trip through shared
// memory, which is why this is mma.sync and not tcgen05 (whose operands must be staged in
// shared memory in canonical layout at 2 B per code).
//
// Structure (one CTA = 4 consumer warps + a producer warp + a query warp, two CTAs per SM,
// persistent):
//   * a small kernel first sorts every row's blocks by rung; work items are (cache row, run of
//     up to 32 entries of that sorted list), numbered chunk-major and handed out by an atomic
//     counter; every item ends in one (m, l, o) record per consumer warp and query head;
//   * the producer warp streams each block's bytes and its four scale planes into a byte
//     ring in shared memory with cp.async.bulk + mbarrier (non-multicast), several blocks
//     ahead of the consumers, and announces every item one item early;
//   * the query warp turns the next item's query rows into MMA A-fragment planes (double
//     buffered), so the consumers never stop at an item boundary;
//   * consumer warps work in pairs: a pair takes every second block of the stream and each of
//     its warps one half of the block's tokens, with a private online softmax.  A block is
//     therefore resident for half as long, which doubles the part of the ring that is free
//     for copies in flight.  Nothing is merged inside the CTA: the combine kernel merges the
//     per-warp records together with the split records.
//
// Arithmetic.  Integer codes are fed to the MMA as fp16 values from the LINEAR range of the
// format: bit patterns 0..2047 (subnormals and the first binade) are worth pattern * 2^-24, so a
// code masked out of the packed word already is the number "code * 2^k * 2^-24" and unpacking
// needs no int->float conversion.  The tensor core aligns the products of a dot product by their
// nominal exponents, so a code sitting in the low mantissa bits wastes that many bits of the
// accumulation window (measured: 2-bit codes at bit 0 lose ~10 bits); codes are therefore
// placed as high in the linear range as a single shift allows (bits 8-9 / 6-7 for 2-bit,
// 7-10 / 3-6 for 4-bit, 0-7 for 8-bit) and the power of two is folded into the query planes.
// De-quantisation is hoisted out of the contraction:
//   q . (c*step + lo) = (q*step) . c + q . lo        (per token group, per channel)
//   p . (c*step + lo) = (p*step) . c + p . lo        (per token, per channel group)
// The small operands q*step and p*step are split into fp16 hi + lo halves that ride in the
// otherwise unused MMA rows 8..15 (the GQA group is at most 8 heads), giving ~22 significant
// bits; the lo terms ride along as one more n-tile on each side.  Accumulation is fp32 throughout.
#pragma once

#include "gkv_common.cuh"

namespace gkv {
namespace mma {

#ifndef GKV_NW
#define GKV_NW 4          // consumer warps per CTA
#endif
#ifndef GKV_CTAS
#define GKV_CTAS 2        // CTAs per SM
#endif
#ifndef GKV_K_FETCH
#define GKV_K_FETCH 16    // widest shared-memory load used for a lane's codes of a K row (4, 8 or 16 bytes)
#endif
#ifndef GKV_RING_KB
#define GKV_RING_KB 71    // byte ring per CTA
#endif
constexpr int kConsumerWarps = GKV_NW;
constexpr int kCtasPerSM = GKV_CTAS;
constexpr int kConsumers = kConsumerWarps * 32;
#if GKV_NW == 4 && GKV_CTAS == 2 && !defined(GKV_NO_REG_SHIFT) && !defined(GKV_REG_SHIFT)
#define GKV_REG_SHIFT 1
#endif
#ifdef GKV_REG_SHIFT
// Register re-allocation between warpgroups (setmaxnreg): the CTA is two full warpgroups, the
// consumers' and a helper one (producer warp, query warp, two warps that leave at once); the
// helpers hand most of their registers to the consumers (200 instead of 168 each: enough to keep
// the whole K loop of a unit unrolled with its loads in flight, measured +4 %).  Launched with 128
// registers per thread, two CTAs per SM.
constexpr int kThreads = kConsumers + 128;
#ifndef GKV_HELPER_REGS
#define GKV_HELPER_REGS 56
#endif
constexpr int kHelperRegs = GKV_HELPER_REGS, kConsumerRegs = 256 - GKV_HELPER_REGS;   // 128 * (helper + consumer) = 256 threads * 128 registers at launch
static_assert(kConsumerWarps == 4, "the consumers must be exactly one warpgroup");
#else
constexpr int kThreads = kConsumers + 64;    // + producer warp + query warp
#endif
static_assert(kConsumerWarps % 2 == 0, "consumer warps work in pairs");
constexpr int kNSlot = kConsumerWarps <= 4 ? 16 : 32;   // descriptor slots (blocks in flight per CTA)
constexpr uint32_t kRingBytes = GKV_RING_KB * 1024;
constexpr int kItemSlots = 4;           // item descriptors in flight: finishing, current, announced, spare
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // every wait gives up after ~1 s, flags the error, returns

struct Desc {           // one block in the ring
    uint32_t off;       // byte offset of the block in the ring
    int32_t level;      // 0 = nothing to do (padding slot)
    int32_t nvalid;
    int32_t pad;
};

struct ItemDesc {       // one work item; published one item ahead of its blocks (ring of kItemSlots)
    int32_t item;
    int32_t row;
    int32_t end_seq;    // the item's blocks are the stream positions up to (not including) this one
    int32_t exit;
};

struct Params {
    const float* q;
    const uint8_t* data;
    const int64_t* offs;
    const __half* klo;
    const __half* kstep;
    const __half* vlo;
    const __half* vstep;
    const int32_t* level;
    const int32_t* valid;
    const uint4* plan;  // (metadata rows, nb) block entries of every row sorted by rung, from plan_kernel
    float* part;        // (rows, items per row, consumer warps, rep, D+2)
    int* counter;       // work-item counter (zeroed before launch)
    int* status;        // error word (zeroed before launch)
    int B, Hq, Hkv, nb, rep;
    int chunk;          // blocks per item for the first nbig chunks of a row's sorted list ...
    int chunk2, nbig;   // ... and for the chunks after them (smaller items at the end trim the tail of the grid)
    int items_per_row, items;
    int per_row_meta;
    int rows;
    int64_t stride_bh;
};

// ---- PTX wrappers --------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: false if the phase did not complete within kWaitLimitNs of wall time.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t a = smem_u32(bar);
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(a), "r"(parity) : "memory");
        if (ok) return true;
#ifndef GKV_NO_BACKOFF
        if (spin > 2) __nanosleep(spin < 64 ? 32 : 256);      // back off: spinning warps steal issue slots
#endif
        if ((spin & 63u) == 63u) {
            const unsigned long long now = global_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitLimitNs) return false;
        }
    }
}
// Shared-memory loads by 32-bit shared address (keeps the address arithmetic in 32 bits).
__device__ __forceinline__ uint32_t lds_u8(uint32_t a) { uint32_t v; asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u16(uint32_t a) { uint32_t v; asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint32_t lds_u32(uint32_t a) { uint32_t v; asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a)); return v; }
__device__ __forceinline__ uint2 lds_v2(uint32_t a) { uint2 v; asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a)); return v; }
__device__ __forceinline__ uint4 lds_v4(uint32_t a) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a)); return v; }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
// Arrives on the barrier (without adding to its expected count) when all earlier cp.async of this thread have landed.
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// (x*y) as fp16 hi + lo, x given as fp16 hi/lo halves, y exact fp16: hi = rn(xh*y),
// lo = rn(xl*y + (xh*y - hi)); the inner difference is exact in an fp16 FMA.
__device__ __forceinline__ void mul_split(uint32_t xh, uint32_t xl, uint32_t y, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __hmul2(u32_as_h2(xh), u32_as_h2(y));
    const __half2 e = __hfma2(u32_as_h2(xh), u32_as_h2(y), __hneg2(h));
    hi = h2_as_u32(h);
    lo = h2_as_u32(__hfma2(u32_as_h2(xl), u32_as_h2(y), e));
}

// Two fp32 values -> packed fp16 hi pair and residual lo pair (element 0 in the low half).
__device__ __forceinline__ void split_f16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __half2 h = __floats2half2_rn(x0, x1);
    const float2 hf = __half22float2(h);
    hi = h2_as_u32(h);
    lo = h2_as_u32(__floats2half2_rn(x0 - hf.x, x1 - hf.y));
}
__device__ __forceinline__ void split_bf16x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x0, x1);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x0 - hf.x, x1 - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
}

// ---- channel arrangement of the QK contraction -----------------------------------------------
// Thread t of a quad owns DT = D/4 consecutive channels of a token row.  MMA k-step s, slot e
// (e = 0,1 -> first B register, e = 2,3 -> second) maps to channel DT*t + arr_chan(bits, s, e);
// the maps follow the cheapest shift-and-mask unpack of each code width (one 32-bit AND yields
// the two codes that sit 16 bits apart).  arr_scale is the exact power of two folded into the
// prepared query so that every slot of a rung carries the same weight:
//   4-bit: even nibbles land on bits 3-6 (8c), odd nibbles on bits 7-10 (128c)  -> x16 / x1
//   2-bit: even fields land on bits 8-9 (256c), odd fields on bits 6-7 (64c)    -> x1 / x4
__host__ __device__ constexpr int arr_chan(int bits, int s, int e) {
    return bits == 4   ? 8 * (s >> 1) + 2 * (s & 1) + (e >> 1) + 4 * (e & 1)
           : bits == 2 ? 16 * (s >> 2) + 2 * (s & 3) + (e >> 1) + 8 * (e & 1)
                       : 4 * s + e;   // 8-bit codes and raw bf16
}
__host__ __device__ constexpr float arr_scale(int bits, int e) {
    return bits == 4 ? ((e >> 1) ? 1.f : 16.f) : bits == 2 ? ((e >> 1) ? 4.f : 1.f) : 1.f;
}
// 2^24 / (weight of one code in the linear range) for the K contraction of each rung
__host__ __device__ constexpr float k_unscale(int bits) { return bits == 4 ? 131072.f : bits == 2 ? 65536.f : 16777216.f; }
// V contraction: bit position the codes are brought to, and the weight scale that goes with it
__host__ __device__ constexpr int v_pos(int bits) { return bits == 4 ? 4 : bits == 2 ? 8 : 0; }

template <int D, int G>
struct Cfg {
    static constexpr int DT = D / 4;          // channels per thread in QK
    static constexpr int KS = D / 16;         // QK k-steps
    static constexpr int CH = KS / 2;         // 16-byte chunks of prepared q per thread (2 k-steps each)
    static constexpr int TG = kP / G;         // token groups (K scales)
    static constexpr int NTG = G / 8;         // token n-tiles per token group
    static constexpr int GV = D / G;          // channel groups (V scales)
    static constexpr int NT = G / 8;          // channel n-tiles per channel group
    static constexpr int NTILE = D / 8;       // output n-tiles
    static constexpr int KSCALE = TG * D * 2; // bytes of klo (or kstep) of one block
    static constexpr int VSCALE = kP * GV * 2;
    // prepared-q planes, in halves: [plane][chunk][lane][8]
    static constexpr int QPLANE = CH * 32 * 8;
    // planes: 0/1 arr8 hi/lo, 2/3 arr4 hi/lo, 4/5 arr2 hi/lo, 6/7 bf16 hi/lo
    static constexpr int QPREP_BYTES = 8 * QPLANE * 2;
    static constexpr int SQ_BYTES = 8 * D * 4;
    static constexpr size_t SMEM = kRingBytes + 2 * (QPREP_BYTES + SQ_BYTES + 64) +
                                   kNSlot * sizeof(Desc) + 2 * kNSlot * 8 + kItemSlots * sizeof(ItemDesc) +
                                   (2 * kItemSlots + 2) * 8 + 32 * 16 + 64;
    static_assert(D % 32 == 0 && (G == 16 || G == 32 || G == 64) && D % G == 0, "unsupported shape");
};

template <int D, int G>
struct Smem {
    using C = Cfg<D, G>;
    uint8_t* ring;
    __half* qprep;         // [2] prepared-query planes (item parity)
    float* sq;             // [2][8][D] raw query (fp32, softmax scale included)
    float* sf;             // [2][16]: per-head factor 2^-eq * log2(e), then 2^eq
    Desc* desc;
    uint64_t* full;
    uint64_t* empty;
    ItemDesc* item;        // [kItemSlots]
    uint64_t* item_full;   // [kItemSlots] producer -> query warp and consumers
    uint64_t* item_empty;  // [kItemSlots] one arrival per consumer warp that finished the item
    uint64_t* qready;      // [2] query warp -> consumers
    uint4* meta_tab;       // [32] block table of the producer's current item
    __device__ explicit Smem(uint8_t* base) {
        ring = base;
        qprep = reinterpret_cast<__half*>(base + kRingBytes);
        sq = reinterpret_cast<float*>(base + kRingBytes + 2 * C::QPREP_BYTES);
        sf = sq + 2 * 8 * D;
        desc = reinterpret_cast<Desc*>(sf + 32);
        full = reinterpret_cast<uint64_t*>(desc + kNSlot);
        empty = full + kNSlot;
        item_full = empty + kNSlot;
        item_empty = item_full + kItemSlots;
        qready = item_empty + kItemSlots;
        item = reinterpret_cast<ItemDesc*>(qready + 2);
        meta_tab = reinterpret_cast<uint4*>(item + kItemSlots);
    }
};

// ================================ producer ====================================================
// Work items are numbered chunk-major: item = chunk * rows + row, and a chunk is a run of p.chunk
// consecutive entries of the row's rung-sorted block list.  The whole grid therefore walks the
// ladder together — all bf16 blocks first, the centroids last: the warps that share an SM run
// the same unpack code at the same time (with the rungs interleaved the kernel spent ~15 % of
// its time refetching instructions), and the cheapest items come last, which trims the tail.
struct Span { int row, b_lo, nblk; };
__device__ __forceinline__ Span span_of(const Params& p, int it) {
    if (it >= p.items) return Span{0, 0, 0};
    const int c = it / p.rows;
    const int b_lo = c < p.nbig ? c * p.chunk : p.nbig * p.chunk + (c - p.nbig) * p.chunk2;
    return Span{it % p.rows, b_lo, min(c < p.nbig ? p.chunk : p.chunk2, p.nb - b_lo)};     // nblk <= 32
}

// ---- rung-sorted block lists -----------------------------------------------------------------------
// One CTA per metadata row: a stable counting sort of the row's blocks by rung (16, 8, 4, 2,
// centroid, then blocks with nothing to do).  An entry is everything the producer needs to know
// about a block: byte offset in the row (64 bit), level | nvalid << 8 (level 0: skip), block index.  Every thread owns a contiguous run of blocks, counts
// its classes, an in-order scan over (class, thread) gives it a write cursor per class, and it
// walks its run once more.  Deterministic: no atomics.  Also clears the workspace header.
constexpr int kPlanMaxThreads = 1024;
__device__ __forceinline__ int rung_class(int lv, int nv) {
    return nv <= 0 ? 5 : lv == 16 ? 0 : lv == 8 ? 1 : lv == 4 ? 2 : lv == 2 ? 3 : lv == 1 ? 4 : 5;
}
__global__ void __launch_bounds__(kPlanMaxThreads) plan_kernel(const int32_t* level, const int32_t* valid, const int64_t* offs,
                                                                uint4* plan, int nb, int* header, int header_ints) {
    // the decode kernel's work counter and status word start at zero
    if (blockIdx.x == 0)
        for (int i = threadIdx.x; i < header_ints; i += blockDim.x) header[i] = 0;
    __shared__ int wsum[kPlanMaxThreads / 32][6];   // per-warp class totals, then their exclusive scan
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarp = blockDim.x >> 5;
    const int32_t* lv = level + (size_t)blockIdx.x * nb;
    const int32_t* nv = valid + (size_t)blockIdx.x * nb;
    const int64_t* of = offs + (size_t)blockIdx.x * nb;
    uint4* out = plan + (size_t)blockIdx.x * nb;
    const int per = (nb + (int)blockDim.x - 1) / (int)blockDim.x;
    const int lo = min(nb, tid * per), hi = min(nb, lo + per);
    int cnt[6] = {0, 0, 0, 0, 0, 0};
    for (int b = lo; b < hi; ++b) {
        const int c = rung_class(lv[b], nv[b]);
#pragma unroll
        for (int k = 0; k < 6; ++k) cnt[k] += (c == k);
    }
    int cur[6];                                     // exclusive prefix inside the warp
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        int x = cnt[k];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int y = __shfl_up_sync(0xffffffffu, x, o);
            if (lane >= o) x += y;
        }
        cur[k] = x - cnt[k];
        if (lane == 31) wsum[warp][k] = x;
    }
    __syncthreads();
    if (tid == 0) {
        int run = 0;
        for (int k = 0; k < 6; ++k)
            for (int w = 0; w < nwarp; ++w) { const int t = wsum[w][k]; wsum[w][k] = run; run += t; }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 6; ++k) cur[k] += wsum[warp][k];
    for (int b = lo; b < hi; ++b) {
        const int l = lv[b], n = min(nv[b], kP);
        const int c = rung_class(l, n);
        const unsigned long long o = (unsigned long long)of[b];
        const uint4 e = make_uint4((uint32_t)o, (uint32_t)(o >> 32), c == 5 ? 0u : ((uint32_t)l | ((uint32_t)n << 8)), (uint32_t)b);
#pragma unroll
        for (int k = 0; k < 6; ++k)
            if (c == k) out[cur[k]++] = e;
    }
}

// The producer warp announces items (one item ahead), and for every block of the current item's
// table (built by the query warp) lane 0 waits for room in the ring, allocates, publishes the slot
// descriptor and starts the bulk copy of the block's bytes; the four scale planes (a few hundred
// bytes each) are then fetched by all 32 lanes with 16-byte asynchronous copies that report to the
// same barrier.  (Five bulk copies per block from one lane cost ~600 cycles of issue time per
// block and made the producer the slowest stage; so did building the tables here.)
template <int D, int G>
__device__ void producer_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    using C = Cfg<D, G>;
    const int lane = threadIdx.x & 31;
    uint32_t head = 0, used = 0;
    int seq_alloc = 0, seq_free = 0;
#ifdef GKV_DBG_TIMING
    long long p_all = clock64(), p_wait = 0, p_issue = 0, p_meta = 0, p_scale = 0, p_n = 0;
#endif

    auto release_oldest = [&]() -> bool {     // all lanes, same result everywhere
        const int s = seq_free % kNSlot;
        if (!mbar_wait(&sm.empty[s], (uint32_t)(seq_free / kNSlot) & 1u)) return false;
        used -= (uint32_t)sm.desc[s].pad;
        ++seq_free;
        return true;
    };
    // Lane 0: announce item number j of this CTA (its descriptor slot is free once the consumers
    // finished item j - kItemSlots, long ago in practice).
    auto announce = [&](int j, int id, const Span& sp, int end_seq) -> bool {
        const int s = j % kItemSlots;
        if (j >= kItemSlots && !mbar_wait(&sm.item_empty[s], (uint32_t)(j / kItemSlots - 1) & 1u)) return false;
        ItemDesc it;
        it.item = id; it.row = sp.row; it.end_seq = end_seq; it.exit = id >= p.items ? 1 : 0;
        sm.item[s] = it;
        mbar_arrive(&sm.item_full[s]);
        return true;
    };

    int item = 0, next_item = 0;
    if (lane == 0) { item = atomicAdd(p.counter, 1); next_item = atomicAdd(p.counter, 1); }
    item = __shfl_sync(0xffffffffu, item, 0);
    next_item = __shfl_sync(0xffffffffu, next_item, 0);
    bool ok = true;
    if (lane == 0) ok = announce(0, item, span_of(p, item), span_of(p, item).nblk);
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    // Block table of an item: entry `lane` of its run of the row's plan, with the row's base offset
    // added.  The next item's entries are requested at the start of the current item and parked in
    // the table when its last block has been issued, so the global-memory latency is never waited for.
    auto fetch_entry = [&](const Span& sp) -> uint4 {
        uint4 e = make_uint4(0, 0, 0, 0);
        if (lane < sp.nblk) {
            e = p.plan[(size_t)(p.per_row_meta ? sp.row : 0) * p.nb + sp.b_lo + lane];
            const unsigned long long src = (unsigned long long)sp.row * (unsigned long long)p.stride_bh +
                                           (((unsigned long long)e.y << 32) | e.x);
            e.x = (uint32_t)src; e.y = (uint32_t)(src >> 32);
        }
        return e;
    };
    sm.meta_tab[lane] = fetch_entry(span_of(p, item));
    __syncwarp();
    for (int iseq = 0; ok; ++iseq) {
        const bool done = item >= p.items;
        int next2 = 0;
#ifdef GKV_DBG_TIMING
        const long long _pm0 = clock64();
#endif
        const Span cs = span_of(p, item), ns = done ? Span{0, 0, 0} : span_of(p, next_item);
        const int row = cs.row, nblk = cs.nblk;
        if (lane == 0 && !done) {
            next2 = atomicAdd(p.counter, 1);       // item id two ahead
            // the next item goes out now, a whole item early: the query warp needs the time
            ok = announce(iseq + 1, next_item, ns, seq_alloc + nblk + ns.nblk);
        }
        if (done) break;
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        const uint4 next_entry = fetch_entry(ns);
        const uint4* tab = sm.meta_tab;
        const size_t sb0 = (size_t)row * p.nb;
        const uint8_t* klo0 = reinterpret_cast<const uint8_t*>(p.klo) + sb0 * C::KSCALE;
        const uint8_t* kst0 = reinterpret_cast<const uint8_t*>(p.kstep) + sb0 * C::KSCALE;
        const uint8_t* vlo0 = reinterpret_cast<const uint8_t*>(p.vlo) + sb0 * C::VSCALE;
        const uint8_t* vst0 = reinterpret_cast<const uint8_t*>(p.vstep) + sb0 * C::VSCALE;
#ifdef GKV_DBG_TIMING
        p_meta += clock64() - _pm0;
#endif
        for (int j = 0; j < nblk && ok; ++j, ++seq_alloc) {
            // Ring bookkeeping is done by all lanes alike (same values everywhere, so nothing has to be
            // broadcast); only the three operations with side effects are lane 0's.
            const uint4 cur = tab[j];
            const int lvj = (int)(cur.z & 0xffu), orig = (int)cur.w;
            const bool quant = lvj == 8 || lvj == 4 || lvj == 2;
            const uint32_t dbytes = lvj ? 2u * (uint32_t)half_bytes(lvj, D) : 0u;
            const int slot = seq_alloc % kNSlot;
            const uint32_t need = (dbytes + (quant ? 2u * (C::KSCALE + C::VSCALE) : 0u) + 127u) & ~127u;
#ifdef GKV_DBG_TIMING
            const long long _pw0 = clock64();
#endif
            while (ok && seq_alloc - seq_free >= kNSlot) ok = release_oldest();
            const uint32_t waste = (head + need > kRingBytes) ? kRingBytes - head : 0u;
            while (ok && used + waste + need > kRingBytes) ok = release_oldest();
#ifdef GKV_DBG_TIMING
            const long long _pi0 = clock64();
            p_wait += _pi0 - _pw0; ++p_n;
#endif
            if (!ok) break;
            const uint32_t dst = waste ? 0u : head;
            used += waste + need;
            head = dst + need;
            if (head >= kRingBytes) head = 0;
            if (lane == 0) {
                Desc d;
                d.off = dst; d.level = lvj; d.nvalid = (int)((cur.z >> 8) & 0xffu); d.pad = (int32_t)(waste + need);
                sm.desc[slot] = d;
                const uint8_t* src = p.data + (((unsigned long long)cur.y << 32) | cur.x);
                uint8_t* d0 = sm.ring + dst;
#ifdef GKV_DBG_NOLOAD
                if (true) { mbar_arrive(&sm.full[slot]); } else
#endif
                if (lvj && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                    mbar_arrive_tx(&sm.full[slot], dbytes);
                    bulk_g2s(d0, src, dbytes, &sm.full[slot]);
                } else {
                    // block start not 16-byte aligned (a cache row at an odd address): no bulk copy,
                    // this lane copies the bytes by hand
                    for (uint32_t i = 0; i < dbytes; ++i) d0[i] = src[i];
                    __threadfence_block();
                    mbar_arrive(&sm.full[slot]);
                }
            }
#ifdef GKV_DBG_TIMING
            const long long _ps0 = clock64();
            p_issue += _ps0 - _pi0;
#endif
#ifndef GKV_DBG_NOLOAD
            if (quant) {
                const uint32_t sdst = smem_u32(sm.ring) + dst + dbytes;
                const size_t ko = (size_t)orig * C::KSCALE, vo = (size_t)orig * C::VSCALE;
                constexpr int K = C::KSCALE, V = C::VSCALE;
#pragma unroll
                for (int o0 = 0; o0 < 2 * (K + V); o0 += 512) {
                    const int o = o0 + lane * 16;
                    if (o < 2 * (K + V)) {
                        const uint8_t* src = o < K ? klo0 + ko + o : o < 2 * K ? kst0 + ko + (o - K)
                                           : o < 2 * K + V ? vlo0 + vo + (o - 2 * K) : vst0 + vo + (o - 2 * K - V);
                        cp_async16(sdst + (uint32_t)o, src);
                    }
                }
            }
#endif
            cp_async_arrive(&sm.full[slot]);                    // one arrival per lane once its copies have landed
#ifdef GKV_DBG_TIMING
            p_scale += clock64() - _ps0;
#endif
        }
        if (!ok) break;
        __syncwarp();
        sm.meta_tab[lane] = next_entry;
        __syncwarp();
        item = next_item;
        next_item = __shfl_sync(0xffffffffu, next2, 0);
    }
#ifdef GKV_DBG_TIMING
    if (lane == 0) {
        unsigned long long* dbg = reinterpret_cast<unsigned long long*>(p.counter) + 4;
        atomicAdd(dbg + 0, (unsigned long long)(clock64() - p_all));
        atomicAdd(dbg + 1, (unsigned long long)p_wait);
        atomicAdd(dbg + 2, (unsigned long long)p_issue);
        atomicAdd(dbg + 3, (unsigned long long)p_meta);
        atomicAdd(dbg + 4, (unsigned long long)p_scale);
        atomicAdd(dbg + 5, (unsigned long long)p_n);
    }
#endif
    if (!ok && lane == 0) {
        atomicExch(p.status, 1);
        atomicExch(abort_flag, 1);
    }
}

// ================================ consumers ===================================================
template <int D, int G>
struct WarpState {
    using C = Cfg<D, G>;
    float o[C::NTILE][4];   // rows r (c0,c1) and r+8 (c2,c3) of every output n-tile, scaled 2^-16
    float ob[4];            // sum_j p_j * vlo[j][cg], scaled 2^8
    float m;                // running max of head r (log2 domain), replicated over the quad
    float l;              // this thread's share of the running sum
};

// ================================ query warp ==================================================
// For every announced item: the row's query heads as fp32 (for the centroid path), a per-head
// power-of-two scale, and the MMA A-fragment planes of every channel arrangement, into the
// buffer of the item's parity.  Runs one item ahead of the consumers.
template <int D, int G>
__device__ void query_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    using C = Cfg<D, G>;
    const int lane = threadIdx.x & 31;
    int code = 0;
    for (int j = 0;; ++j) {
        const int s = j % kItemSlots, ib = j & 1;
        if (!mbar_wait(&sm.item_full[s], (uint32_t)(j / kItemSlots) & 1u)) { code = 7; break; }
        const ItemDesc it = sm.item[s];
        if (it.exit) return;
        // the query buffer was last used by item j-2: wait until every consumer warp has left it
        if (j >= 2 && !mbar_wait(&sm.item_empty[(j - 2) % kItemSlots], (uint32_t)((j - 2) / kItemSlots) & 1u)) { code = 8; break; }
        float* sq = sm.sq + ib * 8 * D;
        float* sf = sm.sf + ib * 16;
        __half* qp = sm.qprep + (size_t)ib * (C::QPREP_BYTES / 2);
        const int b = it.row / p.Hkv, hk = it.row % p.Hkv;
        const float* q = p.q + ((size_t)b * p.Hq + (size_t)hk * p.rep) * D;
        for (int i = lane; i < 8 * D; i += 32) sq[i] = (i / D) < p.rep ? q[i] : 0.f;
        __syncwarp();
        // per-head power-of-two scale bringing max|q| into [8, 16)
        for (int h = 0; h < 8; ++h) {
            float mx = 0.f;
            for (int d = lane; d < D; d += 32) mx = fmaxf(mx, fabsf(sq[h * D + d]));
#pragma unroll
            for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            int eq = 0;
            if (mx > 0.f && mx < INFINITY) eq = 3 - ilogbf(mx);
            eq = max(-100, min(100, eq));
            if (lane == 0) {
                sf[h] = ldexpf(1.4426950408889634f, -eq);
                sf[8 + h] = ldexpf(1.0f, eq);
            }
        }
        __syncwarp();
        // which rungs does the item hold?  (its run of the sorted plan; usually one or two)
        const Span sp = span_of(p, it.item);
        int lvl = 0;
        if (lane < sp.nblk) lvl = (int)(p.plan[(size_t)(p.per_row_meta ? sp.row : 0) * p.nb + sp.b_lo + lane].z & 0xffu);
        const bool need8 = __any_sync(0xffffffffu, lvl == 8), need4 = __any_sync(0xffffffffu, lvl == 4);
        const bool need2 = __any_sync(0xffffffffu, lvl == 2), need16 = __any_sync(0xffffffffu, lvl == 16);
        // This lane writes its own fragment lane of every chunk: 8 halves (two k-steps x four slots)
        // per plane and chunk, as one 16-byte store.  Only the arrangements of rungs that occur.
        {
            const int r = lane >> 2, t = lane & 3;
            const float sc = sf[8 + r];
            const float* qr = sq + r * D + C::DT * t;
#pragma unroll
            for (int a = 0; a < 4; ++a) {
                const int bits = a == 0 ? 8 : a == 1 ? 4 : a == 2 ? 2 : 16;
                const bool need = a == 0 ? need8 : a == 1 ? need4 : a == 2 ? need2 : need16;
                if (!need) continue;
#pragma unroll 1
                for (int i = 0; i < C::CH; ++i) {
                    uint32_t hi[4], lo[4];
#pragma unroll
                    for (int jp = 0; jp < 4; ++jp) {            // halves 2jp, 2jp+1: k-step 2i + (jp >> 1), slots 2(jp & 1) + {0, 1}
                        const int ks = 2 * i + (jp >> 1), e0 = 2 * (jp & 1);
                        const float x0 = qr[arr_chan(bits, ks, e0)] * sc * arr_scale(bits, e0);
                        const float x1 = qr[arr_chan(bits, ks, e0 + 1)] * sc * arr_scale(bits, e0 + 1);
                        if (a < 3) split_f16x2(x0, x1, hi[jp], lo[jp]);
                        else split_bf16x2(x0, x1, hi[jp], lo[jp]);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(qp + (size_t)(2 * a) * C::QPLANE + ((size_t)i * 32 + lane) * 8);
                    dst[0] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
                    dst[C::QPLANE / 8] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.qready[ib]);
    }
    if (lane == 0) {
        atomicExch(p.status, code);
        atomicExch(abort_flag, 1);
    }
}

// The blocks are processed in UNITS of G tokens (one token group of the K scales): scores of
// the unit, online-softmax update, value product of the unit.  Loops over the contraction
// (chunks of two k-steps on the K side, 16-token k-steps on the V side) are real loops, not
// unrolled: the fully unrolled kernel was 130 KB of code and spent most of its time waiting
// for instruction fetches.  All shared-memory operands are addressed by 32-bit shared
// addresses built from one per-thread base plus compile-time offsets.
template <int D, int G>
struct Unit {
    static constexpr int U = G;          // tokens
    static constexpr int NU = G / 8;     // token n-tiles
    static constexpr int KU = G / 16;    // PV k-steps
    static constexpr int ZN = G / 4;     // scores held per thread
};

// Inside every 8-token n-tile of a quantised block, score column c stands for token
// token_of_column(c) = (0, 1, 3, 2, 4, 5, 7, 6)[c].  On the K side that is just which row a lane
// reads; on the V side it makes the four lanes of a quad read token rows of alternating parity
// (t, t+1 swapped for odd t), which halves the bank conflicts of the 4-bit value rows, while a
// lane's two tokens of a k-pair stay neighbours so their scales still come from one load.
__device__ __forceinline__ int token_of_column(int c) { return c ^ ((c >> 1) & 1); }

template <int D, int G>
struct Ctx {                             // per-thread constants of the consumer role
    uint32_t qprep;                      // shared address of this lane's first prepared-query chunk (plane 0)
    uint32_t sq;                         // shared address of the fp32 query rows
    float f;                             // 2^-eq * log2(e) of head r
    int r, t, lane;
};

template <int D, int G>
__device__ __forceinline__ uint4 qchunk(const Ctx<D, G>& c, int plane, int i) {
    return lds_v4(c.qprep + (uint32_t)(plane * Cfg<D, G>::QPLANE * 2 + i * 512));
}

// ---- K side of one unit of a quantised block: scores in the log2 domain ---------------------------
template <int D, int G, int BITS>
__device__ __forceinline__ void scores_unit(const Ctx<D, G>& c, uint32_t blk, int tg, float (&z)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr int RB = D * BITS / 8;                     // bytes per token row
    constexpr int TB = RB / 4;                           // bytes per thread per row
    constexpr int plane = BITS == 8 ? 0 : BITS == 4 ? 2 : 4;
    const uint32_t nat = blk + (uint32_t)(2 * (kP * RB) + C::KSCALE + (tg * D + C::DT * c.t) * 2);
    // The thread's codes of a token row are fetched with the widest load that fits (all chunks at
    // once for 4- and 2-bit codes): a quarter warp then reads whole rows side by side, free of the
    // bank conflicts that one 4-byte load per chunk had (rows are 32-128 bytes apart).
    constexpr int CB = TB / C::CH;                       // code bytes per thread, row and chunk
    constexpr int LB0 = TB < GKV_K_FETCH ? TB : GKV_K_FETCH;
    constexpr int LB = LB0 < CB ? CB : LB0;              // bytes per fetch (at least one chunk)
    constexpr int CG = LB / CB;                          // chunks per fetch
    constexpr int LW = LB / 4;
    static_assert(LB >= 4 && C::CH % CG == 0, "unsupported shape");
    const uint32_t row0 = blk + (uint32_t)((tg * UU::U + token_of_column(c.r)) * RB + c.t * TB);

    float acc[UU::NU][4];
#pragma unroll
    for (int n = 0; n < UU::NU; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    // q . klo of this token group rides along as one more n-tile whose eight columns all carry the
    // group's klo (so every thread ends up with its own head's value, no shuffle); two accumulators,
    // one per k-step of a chunk, keep the MMAs independent.
    float bias0[4] = {0.f, 0.f, 0.f, 0.f}, bias1[4] = {0.f, 0.f, 0.f, 0.f};
#ifndef GKV_K_ROLLED
#pragma unroll
#else
#pragma unroll 1
#endif
    for (int g = 0; g < C::CH / CG; ++g) {
        uint32_t W[UU::NU][LW];
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) {
            const uint32_t src = row0 + (uint32_t)(g * LB + n * 8 * RB);
            if (LW == 4) { const uint4 v = lds_v4(src); W[n][0] = v.x; W[n][1 % LW] = v.y; W[n][2 % LW] = v.z; W[n][3 % LW] = v.w; }
            else if (LW == 2) { const uint2 v = lds_v2(src); W[n][0] = v.x; W[n][1 % LW] = v.y; }
            else W[n][0] = lds_u32(src);
        }
#pragma unroll
        for (int ii = 0; ii < CG; ++ii) {                // two k-steps at a time
            const int i = g * CG + ii;
            const uint4 qh = qchunk(c, plane, i), ql = qchunk(c, plane + 1, i);
            uint32_t sp[4], lp[4];                       // kstep / klo pairs of k-steps 2i and 2i+1 in this arrangement
            if (BITS == 8) {
                const uint4 v = lds_v4(nat + 16 * i), l = lds_v4(nat - C::KSCALE + 16 * i);
                sp[0] = v.x; sp[1] = v.y; sp[2] = v.z; sp[3] = v.w;
                lp[0] = l.x; lp[1] = l.y; lp[2] = l.z; lp[3] = l.w;
            } else if (BITS == 4) {                      // s = 2x+y with x = i: words 4i+y, 4i+y+2
                const uint4 v = lds_v4(nat + 16 * i), l = lds_v4(nat - C::KSCALE + 16 * i);
                sp[0] = prmt(v.x, v.z, 0x5410); sp[1] = prmt(v.x, v.z, 0x7632);
                sp[2] = prmt(v.y, v.w, 0x5410); sp[3] = prmt(v.y, v.w, 0x7632);
                // the query plane carries x16 on slots 0,1 (arr_scale): take it back out of klo
                const __half2 k16 = __float2half2_rn(0.0625f);
                lp[0] = h2_as_u32(__hmul2(u32_as_h2(prmt(l.x, l.z, 0x5410)), k16)); lp[1] = prmt(l.x, l.z, 0x7632);
                lp[2] = h2_as_u32(__hmul2(u32_as_h2(prmt(l.y, l.w, 0x5410)), k16)); lp[3] = prmt(l.y, l.w, 0x7632);
            } else {                                     // s = 4x+y: x = i>>1, y = 2(i&1)+{0,1}: words 8x+y, 8x+y+4
                const uint32_t w0 = nat + (uint32_t)(32 * (i >> 1) + 8 * (i & 1));
                const uint2 va = lds_v2(w0), vb = lds_v2(w0 + 16);
                const uint2 la = lds_v2(w0 - C::KSCALE), lb = lds_v2(w0 - C::KSCALE + 16);
                sp[0] = prmt(va.x, vb.x, 0x5410); sp[1] = prmt(va.x, vb.x, 0x7632);
                sp[2] = prmt(va.y, vb.y, 0x5410); sp[3] = prmt(va.y, vb.y, 0x7632);
                // the query plane carries x4 on slots 2,3
                const __half2 k4 = __float2half2_rn(0.25f);
                lp[0] = prmt(la.x, lb.x, 0x5410); lp[1] = h2_as_u32(__hmul2(u32_as_h2(prmt(la.x, lb.x, 0x7632)), k4));
                lp[2] = prmt(la.y, lb.y, 0x5410); lp[3] = h2_as_u32(__hmul2(u32_as_h2(prmt(la.y, lb.y, 0x7632)), k4));
            }
            mma_f16(bias0, qh.x, ql.x, qh.y, ql.y, lp[0], lp[1]);
            mma_f16(bias1, qh.z, ql.z, qh.w, ql.w, lp[2], lp[3]);
            uint32_t a[8];
            mul_split(qh.x, ql.x, sp[0], a[0], a[1]);
            mul_split(qh.y, ql.y, sp[1], a[2], a[3]);
            mul_split(qh.z, ql.z, sp[2], a[4], a[5]);
            mul_split(qh.w, ql.w, sp[3], a[6], a[7]);
            uint32_t bb[UU::NU][4];                      // B registers of k-steps 2i (0,1) and 2i+1 (2,3)
#pragma unroll
            for (int n = 0; n < UU::NU; ++n) {
                if (BITS == 8) {
                    const uint32_t wx = W[n][(2 * ii) % LW], wy = W[n][(2 * ii + 1) % LW];
                    bb[n][0] = prmt(wx, 0u, 0x4140); bb[n][1] = prmt(wx, 0u, 0x4342);
                    bb[n][2] = prmt(wy, 0u, 0x4140); bb[n][3] = prmt(wy, 0u, 0x4342);
                } else if (BITS == 4) {
                    const uint32_t w = W[n][ii % LW];
                    const uint32_t u = w << 3, v = w >> 5;
                    bb[n][0] = u & 0x00780078u; bb[n][1] = u & 0x07800780u;
                    bb[n][2] = v & 0x00780078u; bb[n][3] = v & 0x07800780u;
                } else {
                    // fields 4h..4h+3 (and +8) of the word, h = i & 1, brought to bits 8-9 / 6-7
                    const uint32_t w = W[n][(ii >> 1) % LW] >> (8 * (ii & 1));
                    const uint32_t u = w << 4;
                    bb[n][0] = (w << 8) & 0x03000300u; bb[n][1] = u & 0x00C000C0u;
                    bb[n][2] = u & 0x03000300u;        bb[n][3] = w & 0x00C000C0u;
                }
            }
            // k-step major: the two MMAs of an n-tile are NU issues apart, which hides the MMA latency
#pragma unroll
            for (int n = 0; n < UU::NU; ++n) mma_f16(acc[n], a[0], a[1], a[2], a[3], bb[n][0], bb[n][1]);
#pragma unroll
            for (int n = 0; n < UU::NU; ++n) mma_f16(acc[n], a[4], a[5], a[6], a[7], bb[n][2], bb[n][3]);
        }
    }
    const float bg = (bias0[0] + bias0[2]) + (bias1[0] + bias1[2]);      // hi rows + lo rows, both k-steps
#pragma unroll
    for (int n = 0; n < UU::NU; ++n) {
        z[2 * n + 0] = fmaf(acc[n][0] + acc[n][2], k_unscale(BITS), bg) * c.f;
        z[2 * n + 1] = fmaf(acc[n][1] + acc[n][3], k_unscale(BITS), bg) * c.f;
    }
}

template <int D, int G>
__device__ __forceinline__ void scores_unit_bf16(const Ctx<D, G>& c, uint32_t blk, int tg, float (&z)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    const uint32_t row0 = blk + (uint32_t)(((tg * UU::U + c.r) * D + C::DT * c.t) * 2);
    float acc[UU::NU][4];
#pragma unroll
    for (int n = 0; n < UU::NU; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll 1
    for (int i = 0; i < C::CH; ++i) {
        const uint4 qh = qchunk(c, 6, i), ql = qchunk(c, 7, i);
        uint4 w[UU::NU];
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) w[n] = lds_v4(row0 + 16 * i + n * 8 * D * 2);
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) mma_bf16(acc[n], qh.x, ql.x, qh.y, ql.y, w[n].x, w[n].y);
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) mma_bf16(acc[n], qh.z, ql.z, qh.w, ql.w, w[n].z, w[n].w);
    }
#pragma unroll
    for (int n = 0; n < UU::NU; ++n) {
        z[2 * n + 0] = (acc[n][0] + acc[n][2]) * c.f;
        z[2 * n + 1] = (acc[n][1] + acc[n][3]) * c.f;
    }
}

// ---- online-softmax update ---------------------------------------------------------------------
// The running reference m only moves when a score exceeds it by more than kLazy (log2 domain):
// until then weights are taken against the stale reference and may reach 2^kLazy.  That keeps
// the accumulator rescale (one FMUL per output register) off the common path; the fp16 weight
// operands still fit (p * 2^8 * step < 65504 for any step < 16).
constexpr float kLazy = 4.0f;

template <int D, int G>
__device__ __forceinline__ float move_reference(WarpState<D, G>& st, float mx) {
    using C = Cfg<D, G>;
    const bool need = mx > st.m + kLazy || st.m == -INFINITY;   // per head (uniform over the quad)
    if (__any_sync(0xffffffffu, need)) {
        const float mnew = need ? mx : st.m;
        const float corr = ex2(st.m - mnew);          // 0 when st.m = -inf, 1 for the heads that stay
        st.m = mnew;
        st.l *= corr;
#pragma unroll
        for (int n = 0; n < C::NTILE; ++n) {
            st.o[n][0] *= corr; st.o[n][1] *= corr; st.o[n][2] *= corr; st.o[n][3] *= corr;
        }
        st.ob[0] *= corr; st.ob[1] *= corr; st.ob[2] *= corr; st.ob[3] *= corr;
    }
    return st.m;
}

// z: scores of head r for the unit's tokens 8*n + 2t + {0,1} (log2 domain); nrel = valid tokens
// left in this unit (>= 1).  Returns the weights in z.
template <int D, int G, bool PERM>
__device__ __forceinline__ void softmax_unit(const Ctx<D, G>& c, WarpState<D, G>& st, float (&z)[Unit<D, G>::ZN], int nrel) {
    using UU = Unit<D, G>;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < UU::ZN; ++i) {
        const int tok = (i >> 1) * 8 + (PERM ? token_of_column(2 * c.t + (i & 1)) : 2 * c.t + (i & 1));
        if (tok >= nrel) z[i] = -INFINITY;
        mx = fmaxf(mx, z[i]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m = move_reference(st, mx);
    float ls = 0.f;
#pragma unroll
    for (int i = 0; i < UU::ZN; ++i) {
        z[i] = ex2(z[i] - m);
        ls += z[i];
    }
    st.l += ls;
}

// Pairs (x[tok][cg], x[tok+1][cg]) of a (64, GV) fp16 plane at shared address `row` (token `tok`, even);
// `odd` swaps the two tokens of every pair (see token_of_column).
template <int GV>
__device__ __forceinline__ void scale_pairs(uint32_t row, bool odd, uint32_t (&out)[GV]) {
    const uint32_t lo = odd ? 0x1054u : 0x5410u, hi = odd ? 0x3276u : 0x7632u;
    if (GV == 4) {
        const uint4 v = lds_v4(row);
        out[0] = prmt(v.x, v.z, lo); out[1] = prmt(v.x, v.z, hi);
        out[2 % GV] = prmt(v.y, v.w, lo); out[3 % GV] = prmt(v.y, v.w, hi);
    } else if (GV == 2) {
        const uint2 v = lds_v2(row);
        out[0] = prmt(v.x, v.y, lo); out[1 % GV] = prmt(v.x, v.y, hi);
    } else {
        const uint32_t ra = row + (odd ? 2 * GV : 0), rb = row + (odd ? 0 : 2 * GV);
#pragma unroll
        for (int cg = 0; cg < GV; ++cg) out[cg] = lds_u16(ra + 2 * cg) | (lds_u16(rb + 2 * cg) << 16);
    }
}

// ---- V side of one unit of a quantised block -------------------------------------------------------
template <int D, int G, int BITS>
__device__ __forceinline__ void values_unit(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int unit,
                                            float (&pz)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr int RB = D * BITS / 8;
    constexpr int NB = C::NT * BITS;                 // bits one thread reads per token per channel group
    constexpr int POS = v_pos(BITS);                 // codes are brought to bits [POS, POS+BITS) of each half
    constexpr uint32_t MASK = (((1u << BITS) - 1u) << POS) * 0x00010001u;
    constexpr float PSCALE = (float)(256 >> POS);    // weights carry 2^(8-POS) so that every rung adds p*v*2^-16
    const __half2 lo_scale = __float2half2_rn((float)(1 << POS));
    const int tok0 = unit * UU::U + 2 * c.t;         // lower token of this thread's pair in k-step 0
    const bool odd = c.t & 1;                        // odd lanes of a quad take their pair in swapped order
    const uint32_t sw = odd ? RB : 0;
    // codes of (token tok0, channels NT*r .. of group 0); scale rows of token tok0
    uint32_t vrow = blk + (uint32_t)(kP * RB + tok0 * RB + (C::NT * c.r * BITS) / 8);
    uint32_t srow = blk + (uint32_t)(2 * (kP * RB) + 2 * C::KSCALE + tok0 * C::GV * 2);
    constexpr int SUB = ((C::NT * BITS) % 8) ? 1 : 0;  // thread's field starts inside a byte (g=16, 2-bit)
    const int subshift = SUB ? ((C::NT * c.r * BITS) & 7) : 0;
#pragma unroll 1
    for (int ku = 0; ku < UU::KU; ++ku, vrow += 16 * RB, srow += 16 * C::GV * 2) {
        uint32_t ph[2], pl[2];
        split_f16x2(pz[0] * PSCALE, pz[1] * PSCALE, ph[0], pl[0]);
        split_f16x2(pz[2] * PSCALE, pz[3] * PSCALE, ph[1], pl[1]);
#pragma unroll
        for (int j = 0; j + 4 < UU::ZN; ++j) pz[j] = pz[j + 4];       // next k-step's weights move to the front
        uint32_t sa[C::GV], sb[C::GV], la[C::GV], lb[C::GV];
        scale_pairs<C::GV>(srow + C::VSCALE, odd, sa);                // vstep, the lane's token pair of n-tile 2ku
        scale_pairs<C::GV>(srow + C::VSCALE + 8 * C::GV * 2, odd, sb);  // vstep, its pair of n-tile 2ku+1
        scale_pairs<C::GV>(srow, odd, la);                            // vlo
        scale_pairs<C::GV>(srow + 8 * C::GV * 2, odd, lb);
        // p . vlo: column n of this n-tile is channel group n
        {
            uint32_t b0 = 0, b1 = 0;
#pragma unroll
            for (int cg = 0; cg < C::GV; ++cg)
                if (c.r == cg) { b0 = la[cg]; b1 = lb[cg]; }
            if (POS) {                                 // keep the 2^8 scale of the p . vlo accumulator
                b0 = h2_as_u32(__hmul2(u32_as_h2(b0), lo_scale));
                b1 = h2_as_u32(__hmul2(u32_as_h2(b1), lo_scale));
            }
            mma_f16(st.ob, ph[0], pl[0], ph[1], pl[1], b0, b1);
        }
#pragma unroll
        for (int cg = 0; cg < C::GV; ++cg) {
            uint32_t a0, a1, a2, a3;
            mul_split(ph[0], pl[0], sa[cg], a0, a1);
            mul_split(ph[1], pl[1], sb[cg], a2, a3);
            // codes of this thread's NT channels for the four tokens ta, ta+1, tb, tb+1
            uint32_t x[4][(NB + 31) / 32];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t src = vrow + ((k & 1) ? RB - sw : sw) + (uint32_t)(((k & 2) ? 8 : 0) * RB + (G * cg * BITS) / 8);
                if (NB >= 32) {
#pragma unroll
                    for (int w = 0; w < (NB + 31) / 32; ++w) x[k][w] = lds_u32(src + 4 * w);
                } else if (NB == 16) {
                    x[k][0] = lds_u16(src);
                } else {
                    x[k][0] = lds_u8(src) >> subshift;
                }
            }
#pragma unroll
            for (int i = 0; i < C::NT; ++i) {
                const int bp = i * BITS;              // bit position of channel i inside x
                const int w = bp / 32, wb = bp % 32;
                // pack the two tokens' 16-bit halves that contain the field, then shift/mask
                const uint32_t selA = (wb < 16) ? 0x5410u : 0x7632u;
                const uint32_t pa = prmt(x[0][w], x[1][w], selA), pb = prmt(x[2][w], x[3][w], selA);
                const int sh = wb % 16;
                const uint32_t b0 = (sh >= POS ? pa >> (sh - POS) : pa << (POS - sh)) & MASK;
                const uint32_t b1 = (sh >= POS ? pb >> (sh - POS) : pb << (POS - sh)) & MASK;
                mma_f16(st.o[cg * C::NT + i], a0, a1, a2, a3, b0, b1);
            }
        }
    }
}

template <int D, int G>
__device__ __forceinline__ void values_unit_bf16(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int unit,
                                                 float (&pz)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr float kScale = 1.52587890625e-05f;      // 2^-16: same accumulator scale as the code path
    uint32_t vrow = blk + (uint32_t)(kP * D * 2 + ((unit * UU::U + 2 * c.t) * D + C::NT * c.r) * 2);
#pragma unroll 1
    for (int ku = 0; ku < UU::KU; ++ku, vrow += 16 * D * 2) {
        uint32_t a0, a1, a2, a3;
        split_bf16x2(pz[0] * kScale, pz[1] * kScale, a0, a1);
        split_bf16x2(pz[2] * kScale, pz[3] * kScale, a2, a3);
#pragma unroll
        for (int j = 0; j + 4 < UU::ZN; ++j) pz[j] = pz[j + 4];
#pragma unroll
        for (int cg = 0; cg < C::GV; ++cg) {
            uint32_t x[4][C::NT / 2];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t src = vrow + (uint32_t)((((k & 2) ? 8 : 0) + (k & 1)) * D * 2 + G * cg * 2);
#pragma unroll
                for (int w = 0; w < C::NT / 2; ++w) x[k][w] = lds_u32(src + 4 * w);
            }
#pragma unroll
            for (int i = 0; i < C::NT; ++i) {
                const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;
                const uint32_t b0 = prmt(x[0][i / 2], x[1][i / 2], sel);
                const uint32_t b1 = prmt(x[2][i / 2], x[3][i / 2], sel);
                mma_bf16(st.o[cg * C::NT + i], a0, a1, a2, a3, b0, b1);
            }
        }
    }
}

// A block whose tail is not valid: clear what the value product would otherwise read for the
// tokens beyond nvalid (those bytes may hold anything, even NaN patterns), so that the main
// path needs no masks.  Scores of such tokens are forced to -inf by the softmax.
template <int D, int G>
__device__ __forceinline__ void clear_invalid_tail(uint8_t* blk, int level, int nvalid, int lane) {
    using C = Cfg<D, G>;
    if (level == 16) {
        uint32_t* v = reinterpret_cast<uint32_t*>(blk + kP * D * 2 + nvalid * D * 2);
        for (int i = lane; i < (kP - nvalid) * D / 2; i += 32) v[i] = 0u;
    } else {
        const int RB = D * level / 8;
        uint16_t* lo = reinterpret_cast<uint16_t*>(blk + 2 * kP * RB + 2 * C::KSCALE);
        for (int i = nvalid * C::GV + lane; i < kP * C::GV; i += 32) { lo[i] = 0; lo[C::VSCALE / 2 + i] = 0; }
    }
    __syncwarp();
}

// One quantised block, units [u0, u1).
template <int D, int G, int BITS>
__device__ __forceinline__ void quant_block(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int nvalid, int u0, int u1) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    if (u1 <= u0 || nvalid <= u0 * UU::U) return;
#pragma unroll 1
    for (int unit = u0; unit < u1; ++unit) {
        const int nrel = nvalid - unit * UU::U;
        if (nrel <= 0) break;
        float z[UU::ZN];
#ifdef GKV_DBG_NOK
        for (int i = 0; i < UU::ZN; ++i) z[i] = (float)(i + c.r);
#else
        scores_unit<D, G, BITS>(c, blk, unit, z);
#endif
        softmax_unit<D, G, true>(c, st, z, nrel);
#ifndef GKV_DBG_NOV
        values_unit<D, G, BITS>(c, st, blk, unit, z);
#else
        st.l += z[0];
#endif
    }
}

template <int D, int G>
__device__ __forceinline__ void bf16_block(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int nvalid, int u0, int u1) {
    using UU = Unit<D, G>;
#pragma unroll 1
    for (int unit = u0; unit < u1; ++unit) {
        const int nrel = nvalid - unit * UU::U;
        if (nrel <= 0) break;
        float z[UU::ZN];
        scores_unit_bf16(c, blk, unit, z);
        softmax_unit<D, G, false>(c, st, z, nrel);
        values_unit_bf16(c, st, blk, unit, z);
    }
}

// ---- a centroid block: one key and one value stand for nvalid tokens ------------------------------
template <int D, int G>
__device__ __forceinline__ void centroid_block(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int nvalid) {
    using C = Cfg<D, G>;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < C::DT / 8; ++i) {
        const uint4 k8 = lds_v4(blk + (uint32_t)(C::DT * c.t * 2 + 16 * i));
        const uint4 qa = lds_v4(c.sq + (uint32_t)((c.r * D + C::DT * c.t + 8 * i) * 4));
        const uint4 qb = lds_v4(c.sq + (uint32_t)((c.r * D + C::DT * c.t + 8 * i + 4) * 4));
        const float2 k0 = __half22float2(u32_as_h2(k8.x)), k1 = __half22float2(u32_as_h2(k8.y));
        const float2 k2 = __half22float2(u32_as_h2(k8.z)), k3 = __half22float2(u32_as_h2(k8.w));
        s = fmaf(__uint_as_float(qa.x), k0.x, s); s = fmaf(__uint_as_float(qa.y), k0.y, s);
        s = fmaf(__uint_as_float(qa.z), k1.x, s); s = fmaf(__uint_as_float(qa.w), k1.y, s);
        s = fmaf(__uint_as_float(qb.x), k2.x, s); s = fmaf(__uint_as_float(qb.y), k2.y, s);
        s = fmaf(__uint_as_float(qb.z), k3.x, s); s = fmaf(__uint_as_float(qb.w), k3.y, s);
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    const float z = s * 1.4426950408889634f;
    const float m = move_reference(st, z);
    const float w = ex2(z - m) * (float)nvalid;
    if (c.t == 0) st.l += w;
    const float ws = w * 1.52587890625e-05f;
    const uint32_t cv = blk + (uint32_t)(D * 2);
#pragma unroll
    for (int cg = 0; cg < C::GV; ++cg) {
        // this thread's output columns of group cg: channels NT*(2t) .. and NT*(2t+1) .., 2*NT contiguous halves
        uint32_t h[C::NT];
        const uint32_t src = cv + (uint32_t)((G * cg + C::NT * 2 * c.t) * 2);
        if (C::NT == 2) {
            const uint2 v = lds_v2(src);
            h[0] = v.x; h[1 % C::NT] = v.y;
        } else {
#pragma unroll
            for (int w = 0; w < C::NT / 4; ++w) {
                const uint4 v = lds_v4(src + 16 * w);
                h[(4 * w) % C::NT] = v.x; h[(4 * w + 1) % C::NT] = v.y; h[(4 * w + 2) % C::NT] = v.z; h[(4 * w + 3) % C::NT] = v.w;
            }
        }
        // h holds 2*NT halves: first NT for column 2t, next NT for column 2t+1
#pragma unroll
        for (int i = 0; i < C::NT; ++i) {
            const uint32_t w0 = h[i / 2], w1 = h[(C::NT + i) / 2];
            const float v0 = __half2float(__ushort_as_half((uint16_t)((i & 1) ? (w0 >> 16) : (w0 & 0xffffu))));
            const float v1 = __half2float(__ushort_as_half((uint16_t)(((C::NT + i) & 1) ? (w1 >> 16) : (w1 & 0xffffu))));
            st.o[cg * C::NT + i][0] = fmaf(ws, v0, st.o[cg * C::NT + i][0]);
            st.o[cg * C::NT + i][1] = fmaf(ws, v1, st.o[cg * C::NT + i][1]);
        }
    }
}

template <int D, int G>
__device__ void consumer_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    WarpState<D, G> st;
    Ctx<D, G> c;
    c.r = r; c.t = t; c.lane = lane; c.f = 0.f;
    const uint32_t ring = smem_u32(sm.ring);
    // A pair of warps takes every (kConsumerWarps/2)-th block of the stream; inside the block the
    // two warps share out the units of G tokens (a block with a single unit goes to the first).
    constexpr int kPairs = kConsumerWarps / 2;
    constexpr int UPB = kP / UU::U;                 // units per block
    const int pair = warp >> 1, half = warp & 1;
    const int u0 = UPB >= 2 ? half * (UPB / 2) : 0;
    const int u1 = UPB >= 2 ? u0 + UPB / 2 : (half == 0 ? 1 : 0);
    int seq = pair;
    int code = 0;                                   // non-zero: a wait gave up
#ifdef GKV_DBG_TIMING
    long long c_all = clock64(), c_wait = 0, c_comp = 0, c_item = 0, c_n = 0, c_lat = 0, c_latn = 0;
    const unsigned long long t_begin = global_ns();
#endif
    for (int iseq = 0; code == 0; ++iseq) {
        const int is = iseq % kItemSlots, ib = iseq & 1;
#ifdef GKV_DBG_TIMING
        long long _ci0 = clock64();
#endif
        if (!mbar_wait(&sm.item_full[is], (uint32_t)(iseq / kItemSlots) & 1u)) { code = 2; break; }
        const ItemDesc it = sm.item[is];
        if (it.exit) {
#ifdef GKV_DBG_TIMING
            if (lane == 0) {
                unsigned long long* dbg = reinterpret_cast<unsigned long long*>(p.counter) + 12;
                const unsigned long long tnow = global_ns();
                atomicMax(dbg + 8, ~tnow);                        // earliest warp exit (complemented)
                atomicMax(dbg + 9, tnow);                         // latest warp exit
                atomicAdd(dbg + 10, tnow - t_begin);              // sum of warp lifetimes (ns)
                atomicMax(dbg + 11, ~t_begin);                    // earliest start (complemented)
                atomicAdd(dbg + 0, (unsigned long long)(clock64() - c_all));
                atomicAdd(dbg + 1, (unsigned long long)c_wait);
                atomicAdd(dbg + 2, (unsigned long long)c_comp);
                atomicAdd(dbg + 3, (unsigned long long)c_item);
                atomicAdd(dbg + 4, (unsigned long long)c_n);
                atomicAdd(dbg + 5, (unsigned long long)c_lat);
                atomicAdd(dbg + 6, (unsigned long long)c_latn);
            }
#endif
            return;
        }
        if (!mbar_wait(&sm.qready[ib], (uint32_t)(iseq >> 1) & 1u)) { code = 3; break; }
        c.qprep = smem_u32(sm.qprep) + (uint32_t)(ib * C::QPREP_BYTES) + (uint32_t)lane * 16u;
        c.sq = smem_u32(sm.sq) + (uint32_t)(ib * C::SQ_BYTES);
        c.f = sm.sf[ib * 16 + r];
#pragma unroll
        for (int n = 0; n < C::NTILE; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;
        st.ob[0] = st.ob[1] = st.ob[2] = st.ob[3] = 0.f;
        st.m = -INFINITY;
        st.l = 0.f;
#ifdef GKV_DBG_TIMING
        c_item += clock64() - _ci0;
#endif

        for (; seq < it.end_seq; seq += kPairs) {
            const int slot = seq % kNSlot;
#ifdef GKV_DBG_TIMING
            long long _cw0 = clock64();
#endif
            if (!mbar_wait(&sm.full[slot], (uint32_t)(seq / kNSlot) & 1u)) { code = 4; break; }
            const Desc d = sm.desc[slot];
#ifdef GKV_DBG_TIMING
            {
                const long long now = clock64();
                if (now - _cw0 > 400) { c_lat += now - _cw0; ++c_latn; }      // length of the waits that were real waits
                c_wait += now - _cw0; _cw0 = now; ++c_n;
            }
#endif
#ifdef GKV_DBG_NOCOMPUTE
            if (false) {
#else
            if (d.level) {
#endif
                const uint32_t blk = ring + d.off;
                if (d.level == 1) {
                    if (half == 0) centroid_block(c, st, blk, d.nvalid);
                } else {
                    // both warps of the pair clear the tail (same zeros, so the overlap is harmless)
                    if (d.nvalid < kP) clear_invalid_tail<D, G>(sm.ring + d.off, d.level, d.nvalid, lane);
                    if (d.level == 16) bf16_block(c, st, blk, d.nvalid, u0, u1);
                    else if (d.level == 8) quant_block<D, G, 8>(c, st, blk, d.nvalid, u0, u1);
                    else if (d.level == 4) quant_block<D, G, 4>(c, st, blk, d.nvalid, u0, u1);
                    else quant_block<D, G, 2>(c, st, blk, d.nvalid, u0, u1);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[slot]);
#ifdef GKV_DBG_TIMING
            c_comp += clock64() - _cw0;
#endif
        }
        if (code) break;
#ifdef GKV_DBG_TIMING
        _ci0 = clock64();
#endif
        // ---- this warp's record of the item (natural-log domain, like the generic kernel's) ----
        float l = st.l;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const size_t rec_idx = (size_t)it.row * p.items_per_row + (size_t)(it.item / p.rows);
        float* rec = p.part + ((rec_idx * kConsumerWarps + warp) * p.rep + r) * (D + 2);
        const bool live = r < p.rep;
        if (live && t == 0) { rec[0] = st.m * 0.6931471805599453f; rec[1] = l; }
        // p . vlo of channel group cg sits in lane 4r + cg/2, column cg & 1, scaled 2^8
        const float ob_even = st.ob[0] + st.ob[2], ob_odd = st.ob[1] + st.ob[3];
#pragma unroll
        for (int cg = 0; cg < C::GV; ++cg) {
            const float src = (cg & 1) ? ob_odd : ob_even;
            const float bias = __shfl_sync(0xffffffffu, src, (lane & ~3) | (cg >> 1)) * 0.00390625f;
            if (live) {
#pragma unroll
                for (int i = 0; i < C::NT; ++i) {
                    const int n = cg * C::NT + i;
                    rec[2 + G * cg + C::NT * (2 * t) + i] = fmaf(st.o[n][0] + st.o[n][2], 65536.f, bias);
                    rec[2 + G * cg + C::NT * (2 * t + 1) + i] = fmaf(st.o[n][1] + st.o[n][3], 65536.f, bias);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.item_empty[is]);
#ifdef GKV_DBG_TIMING
        c_item += clock64() - _ci0;
#endif
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    }
    if (code && lane == 0) {
        atomicExch(p.status, code);
        atomicExch(abort_flag, 1);
    }
}

template <int D, int G>
__global__ void __launch_bounds__(kThreads, kCtasPerSM) decode_mma_kernel(Params p) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int abort_flag;
    Smem<D, G> sm(smem_raw);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kNSlot; ++s) {
            mbar_init(&sm.full[s], 1 + 32);         // lane 0's arrival (+ bulk-copy bytes) and 32 scale-copy arrivals
            mbar_init(&sm.empty[s], 2);             // the two warps of a pair
        }
        for (int s = 0; s < kItemSlots; ++s) {
            mbar_init(&sm.item_full[s], 1);
            mbar_init(&sm.item_empty[s], kConsumerWarps);
        }
        mbar_init(&sm.qready[0], 1);
        mbar_init(&sm.qready[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
#ifdef GKV_REG_SHIFT
    if (threadIdx.x < kConsumers) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
    if (threadIdx.x >= kConsumers + 64) return;
#endif
    if (threadIdx.x < kConsumers) consumer_loop<D, G>(p, sm, &abort_flag);
    else if (threadIdx.x < kConsumers + 32) producer_loop<D, G>(p, sm, &abort_flag);
    else query_loop<D, G>(p, sm, &abort_flag);
}

}  // namespace mma
}  // namespace gkv
