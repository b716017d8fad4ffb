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
// Structure (one persistent CTA per SM: 12 consumer warps + 2 producer warps + a query warp + a
// scheduler warp):
//   * a small kernel first sorts every cache row's blocks by rung.  A work item is a run of
//     consecutive entries of ONE rung of one row's sorted list (at most kMaxItemBlocks), so an
//     item never mixes rungs: its code path, its query operands and the layout of its
//     accumulators are fixed when it starts.  Items are numbered slot-major (slot * rows + row)
//     and handed out by an atomic counter, so the grid walks the ladder roughly together.  The
//     scheduler warp draws them a few items ahead and parks each item's block table in shared memory;
//   * the blocks of an item alternate between two STREAMS.  Each stream has its own producer
//     warp, its own byte ring in shared memory and three pairs of consumer warps.  The producer
//     streams each block's bytes with one cp.async.bulk and its four scale planes with 16-byte
//     cp.async copies from all lanes, all reporting to the slot's mbarrier;
//   * the query warp turns the next item's query rows into MMA A-fragment planes for the
//     item's rung (double buffered), so the consumers never stop at an item boundary;
//   * a pair of consumer warps takes every third block of its stream and each of its warps
//     one half of the block's tokens, with a private online softmax.  Nothing is merged
//     inside the CTA: the combine kernel merges the per-warp records;
//   * items of centroid blocks (512 bytes each) bypass the rings: the consumer warps read
//     them straight from global memory with one coalesced 16-byte load per lane.
//
// Arithmetic.  Integer codes are fed to the MMA as fp16 values from the LINEAR range of the
// format: bit patterns 0..2047 (subnormals and the first binade) are worth pattern * 2^-24, so a
// code masked out of the packed word already is the number "code * 2^k * 2^-24" and unpacking
// needs no int->float conversion.  The tensor core aligns the products of a dot product by their
// nominal exponents, so a code sitting in the low mantissa bits wastes that many bits of the
// accumulation window (measured: 2-bit codes at bit 0 lose ~10 bits); codes are therefore
// placed as high in the linear range as a single shift allows and the power of two is folded
// into the other operand or into the epilogue.  De-quantisation is hoisted out of the contraction:
//   q . (c*step + lo) = (q*step) . c + q . lo        (per token group, per channel)
//   p . (c*step + lo) = (p*step) . c + p . lo        (per token, per channel group)
// The small operands q*step and p*step are split into fp16 hi + lo halves (~22 significant
// bits); the lo terms ride along as one more MMA tile on each side.  Accumulation is fp32.
//
// Orientation.  QK^T is computed as S[head][token] (A = q*step, hi halves in rows 0-7 and lo halves
// in rows 8-15; B = key codes), which leaves every thread with the weights of its head for the
// token pairs 2t, 2t+1 — exactly a B fragment.  PV is therefore computed TRANSPOSED,
// O^T[channel][head] (A = value codes, fetched with ldmatrix.trans so that a register already
// holds one channel set of two neighbouring tokens; B = p*vstep): 32 accumulator registers per
// thread instead of 64, which is what lets 12 consumer warps share an SM.  With at most four
// query heads per cache row the eight B columns carry (hi, lo) of every head and one MMA does
// both halves; with five to eight heads the hi and lo products are two MMAs into the same
// accumulators.
#pragma once

#include <cuda.h>          // CUtensorMap (the type only; the encoder is looked up at run time)

#include "gkv_common.cuh"

namespace gkv {
namespace mma {

// Tensor maps of the cache bytes, one per rung whose blocks are fetched with a TILED bulk copy: the
// cache is described as a 2-D byte matrix of `w`-byte rows (w = bytes of a token row, at most 128),
// a block is a box of consecutive rows, and the copy engine writes the box into shared memory with
// the 16-byte chunks of every row XOR-permuted by the row number (the hardware swizzle).  Eight
// consecutive token rows then sit in eight different bank groups, which is what makes the
// ldmatrix.trans fetches of the value codes (eight rows per matrix) conflict-free: measured on the
// plain row-major layout, those fetches alone cost 4 to 8 shared-memory wavefronts per matrix.
struct alignas(64) TensorMaps {
    CUtensorMap m[3];   // 0: raw bf16 rows, 1: 8-bit codes, 2: 4-bit codes
    int usable;         // 0: no tiled copies (base pointer not 16-byte aligned, or no encoder): blocks are copied by hand
    int pad[15];
};

constexpr int kConsumerWarps = 12;       // three warpgroups
constexpr int kStreams = 2;              // byte rings / producer warps per CTA
constexpr int kPairsPerStream = kConsumerWarps / 2 / kStreams;
constexpr int kCtasPerSM = 1;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 128;          // + helper warpgroup: producers 0/1, query warp, scheduler warp
// Register re-allocation between warpgroups (setmaxnreg): launched with 128 registers per thread
// (512 threads), the helper warpgroup drops to kHelperRegs and the consumers rise to kConsumerRegs:
// 384 * 152 + 128 * 56 = 65536.
constexpr int kHelperRegs = 56, kConsumerRegs = 152;
#ifndef GKV_K_FETCH
#define GKV_K_FETCH 16    // widest shared-memory load used for a lane's codes of a K row (4, 8 or 16 bytes)
#endif
#ifndef GKV_RING_KB
#define GKV_RING_KB 100   // byte ring per stream
#endif
#ifndef GKV_NSLOT
#define GKV_NSLOT 16
#endif
constexpr int kNSlot = GKV_NSLOT;        // descriptor slots (blocks in flight) per stream
constexpr uint32_t kRingBytes = GKV_RING_KB * 1024;
constexpr int kMaxItemBlocks = 128;      // blocks per work item (the item's block table in shared memory)
constexpr int kMaxCentroidItemBlocks = 64;   // centroid items are held in registers by the warps that read them: shorter
constexpr int kMinItemBlocks = kConsumerWarps / 2;   // one block per pair
constexpr int kItemSlots = 4;            // item descriptors in flight: finishing, current, announced, spare
#ifndef GKV_WAIT_LIMIT_NS
#define GKV_WAIT_LIMIT_NS 1000000000ull
#endif
constexpr unsigned long long kWaitLimitNs = GKV_WAIT_LIMIT_NS;  // every wait gives up after ~1 s, flags the error, returns
constexpr int kPlanTabInts = 8;          // per metadata row: start of each rung class in the sorted list (6), nb, padding

struct Desc {           // one block in a ring
    uint32_t off;       // byte offset of the block in the ring
    int32_t nvalid;
    int32_t pad;        // ring bytes the slot occupies (with alignment and wrap waste)
    int32_t orig;       // the block's index in its cache row (for the per-block softmax mass)
};

struct ItemDesc {       // one work item; published one item ahead of its blocks (ring of kItemSlots)
    int32_t item;       // slot * rows + row
    int32_t row;
    int32_t level;      // rung of every block of the item (16, 8, 4, 2, 1)
    int32_t b_lo;       // first entry of the item in the row's sorted list
    int32_t nblk;
    int32_t first;      // stream of the item's first block (blocks alternate from there)
    int32_t end_seq0;   // per stream: the item's blocks are the stream positions below this
    int32_t end_seq1;
    int32_t exit;
    int32_t pad[3];
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
    const uint4* plan;       // (metadata rows, nb) block entries of every row sorted by rung, from plan_kernel
    const int32_t* plan_tab; // (metadata rows, kPlanTabInts) start of each rung class in that list
    float* part;             // (rows, items per row, consumer warps, rep, D+2)
    float2* mass_part;       // optional (rows, nb, 2 units, rep): (reference, sum of weights against it) per block half and head,
                             // natural-log domain; the by-product from which the per-block softmax mass is made
    int* counter;            // work-item counter (zeroed before launch)
    int* status;             // error word (zeroed before launch)
    int B, Hq, Hkv, nb, rep;
    int chunk;               // blocks per item (the last item of a rung's run may be shorter)
    int items_per_row, items;
    int per_row_meta;
    int rows;
    int paged;               // 1: `data` is a block pool, offs are pool offsets, and the four scale planes of a quantised
                             // block sit right behind its bytes ([klo][kstep][vlo][vstep]); klo..vstep above are unused
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
        // the hint lets the hardware keep the thread suspended for up to ~2 us before it reports "not yet"
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(a), "r"(parity), "r"(2000u) : "memory");
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
// Four 8x8 matrices of 16-bit units, transposed: lane L passes the address of row (L & 7) of matrix
// (L >> 3); thread (r = lane >> 2, t = lane & 3) receives, from each matrix, unit r of rows 2t (low
// half) and 2t+1 (high half).
__device__ __forceinline__ void ldsm_x4_trans(uint32_t a, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
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
// Layout of a rung's block in the ring.  Rungs fetched by a tiled copy are SWIZZLED: byte `off` of the
// block (whose ring address is 1024-byte aligned) lives at off ^ (((off >> 7) & (W/16 - 1)) << 4), W = bytes
// of a tile row (32, 64 or 128) — the 16-byte chunks of a row are permuted by the row's position in
// its group of 128 / W... rows.  W = 0: plain row-major (2-bit codes, and 4-bit codes with 16-channel groups).
template <int D, int G, int BITS>
struct Lay {
    static constexpr int RB = D * BITS / 8;                               // bytes of a token row
    static constexpr bool TILED = BITS == 16 || BITS == 8 || (BITS == 4 && G >= 32);
    static constexpr int W = !TILED ? 0 : RB < 128 ? RB : 128;
    static constexpr uint32_t XMASK = W == 128 ? 7u : W == 64 ? 3u : W == 32 ? 1u : 0u;
    static_assert(!TILED || W >= 32, "tile rows of at least 32 bytes");
};
template <int W>
__device__ __forceinline__ uint32_t swz(uint32_t off) {
    constexpr uint32_t M = W == 128 ? 7u : W == 64 ? 3u : W == 32 ? 1u : 0u;
    return off ^ (((off >> 7) & M) << 4);
}
// XOR term (already shifted to bits 4-6) of a row whose number is r modulo 8, for bytes b of the row
// that do not cross a 128-byte boundary relative to b0.
template <int D, int G, int BITS>
__device__ __forceinline__ uint32_t swz_term(int r, int b0) {
    using L = Lay<D, G, BITS>;
    return ((((uint32_t)r * L::RB + (uint32_t)b0) >> 7) & L::XMASK) << 4;
}

__device__ __forceinline__ void tma_tile_g2s(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
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
// D = A * B (accumulator input zero: the compiler can use the zero register instead of clearing four registers)
__device__ __forceinline__ void mma_f16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ void mma_bf16_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
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

// Head whose scores a thread with row index r (= lane >> 2) holds.  With at most four heads per
// cache row, rows 2h and 2h+1 both carry head h, so that the two threads can feed the hi and the
// lo column of that head in the transposed PV product.
template <bool DUP>
__device__ __forceinline__ int head_of_row(int r) { return DUP ? (r >> 1) : r; }

template <int D, int G>
struct Cfg {
    static constexpr int DT = D / 4;          // channels per thread in QK
    static constexpr int KS = D / 16;         // QK k-steps
    static constexpr int CH = KS / 2;         // 16-byte chunks of prepared q per thread (2 k-steps each)
    static constexpr int TG = kP / G;         // token groups (K scales)
    static constexpr int GV = D / G;          // channel groups (V scales)
    static constexpr int MT = D / 16;         // output m-tiles (16 channels each) of the transposed PV product
    static constexpr int KSCALE = TG * D * 2; // bytes of klo (or kstep) of one block
    static constexpr int VSCALE = kP * GV * 2;
    // prepared-q planes, in halves: [plane][chunk][lane][8]; plane 0 = the A operand (hi, lo, hi, lo) of k-step 2i,
    // plane 1 = that of k-step 2i+1, in the channel arrangement of the item's rung
    static constexpr int QPLANE = CH * 32 * 8;
    static constexpr int QPREP_BYTES = 2 * QPLANE * 2;
    static constexpr int SQ_BYTES = 8 * D * 4;
    static constexpr size_t SMEM = 1024 + kStreams * (size_t)kRingBytes + 2 * (QPREP_BYTES + SQ_BYTES + 64) +
                                   kStreams * kNSlot * (sizeof(Desc) + 16) + kItemSlots * sizeof(ItemDesc) +
                                   (2 * kItemSlots + 2) * 8 + kItemSlots * kMaxItemBlocks * 16 + 128;
    static_assert(D % 32 == 0 && (G == 16 || G == 32 || G == 64) && D % G == 0, "unsupported shape");
};

template <int D, int G>
struct Smem {
    using C = Cfg<D, G>;
    uint8_t* ring;         // [kStreams][kRingBytes]
    __half* qprep;         // [2] prepared-query planes (item parity)
    float* sq;             // [2][8][D] raw query (fp32, softmax scale included)
    float* sf;             // [2][16]: per-head factor 2^-eq * log2(e), then 2^eq
    Desc* desc;            // [kStreams][kNSlot]
    uint64_t* full;        // [kStreams][kNSlot]
    uint64_t* empty;       // [kStreams][kNSlot]
    ItemDesc* item;        // [kItemSlots]
    uint64_t* item_full;   // [kItemSlots] scheduler warp -> producers, query warp and consumers
    uint64_t* item_empty;  // [kItemSlots] one arrival per consumer warp and per producer that is done with the item
    uint64_t* qready;      // [2] query warp -> consumers
    uint4* item_tab;       // [kItemSlots][kMaxItemBlocks] block entries of the announced items (row base offset added)
    __device__ explicit Smem(uint8_t* raw) {
        // the swizzle of the tiled copies is a function of the shared-memory address: rings start on a 1024-byte boundary
        uint8_t* base = raw + ((1024u - (smem_u32(raw) & 1023u)) & 1023u);
        ring = base;
        uint8_t* p = base + kStreams * (size_t)kRingBytes;
        qprep = reinterpret_cast<__half*>(p);               p += 2 * C::QPREP_BYTES;
        sq = reinterpret_cast<float*>(p);                   p += 2 * C::SQ_BYTES;
        sf = reinterpret_cast<float*>(p);                   p += 2 * 16 * 4;
        item_tab = reinterpret_cast<uint4*>(p);             p += kItemSlots * kMaxItemBlocks * 16;
        item = reinterpret_cast<ItemDesc*>(p);              p += kItemSlots * sizeof(ItemDesc);
        desc = reinterpret_cast<Desc*>(p);                  p += kStreams * kNSlot * sizeof(Desc);
        full = reinterpret_cast<uint64_t*>(p);              p += kStreams * kNSlot * 8;
        empty = reinterpret_cast<uint64_t*>(p);             p += kStreams * kNSlot * 8;
        item_full = reinterpret_cast<uint64_t*>(p);         p += kItemSlots * 8;
        item_empty = reinterpret_cast<uint64_t*>(p);        p += kItemSlots * 8;
        qready = reinterpret_cast<uint64_t*>(p);
    }
};

// ---- rung-sorted block lists -----------------------------------------------------------------------
// One CTA per metadata row: a stable counting sort of the row's blocks by rung (16, 8, 4, 2,
// centroid, then blocks with nothing to do).  An entry is everything the producer needs to know
// about a block: byte offset in the row (64 bit), level | nvalid << 8 (level 0: skip), block index.
// Every thread owns a contiguous run of blocks, counts its classes, an in-order scan over
// (class, thread) gives it a write cursor per class, and it walks its run once more.  Deterministic:
// no atomics.  The start of every class in the list goes to the row's table.  Also clears the
// workspace header when given one.
constexpr int kPlanMaxThreads = 1024;
__device__ __forceinline__ int rung_class(int lv, int nv) {
    return nv <= 0 ? 5 : lv == 16 ? 0 : lv == 8 ? 1 : lv == 4 ? 2 : lv == 2 ? 3 : lv == 1 ? 4 : 5;
}
__global__ void __launch_bounds__(kPlanMaxThreads) plan_kernel(const int32_t* level, const int32_t* valid, const int64_t* offs,
                                                                uint4* plan, int32_t* plan_tab, int nb, int* header,
                                                                int header_ints) {
    // the decode kernel's work counter and status word start at zero
    if (blockIdx.x == 0 && header)
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
        int32_t* tab = plan_tab + (size_t)blockIdx.x * kPlanTabInts;
        for (int k = 0; k < 6; ++k) {
            tab[k] = run;                           // class k occupies [tab[k], tab[k+1]) of the list
            for (int w = 0; w < nwarp; ++w) { const int t = wsum[w][k]; wsum[w][k] = run; run += t; }
        }
        tab[6] = nb; tab[7] = 0;
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

// ================================ producers ===================================================
// Item `id` = slot * rows + row.  Slot s of a row is the s-th chunk when each rung's run of the
// row's sorted list is cut into chunks of p.chunk blocks; slots beyond the row's last chunk are
// empty (rows have a fixed number of slots, enough for any mix of rungs).
struct Span { int row, level, b_lo, nblk; };
__device__ __forceinline__ Span span_of(const Params& p, int id) {
    Span sp{0, 0, 0, 0};
    if (id >= p.items) return sp;
    int slot = id / p.rows;
    sp.row = id % p.rows;
    const int32_t* tab = p.plan_tab + (size_t)(p.per_row_meta ? sp.row : 0) * kPlanTabInts;
    // Items are handed out slot by slot over all rows, so at any moment the whole grid works on the same
    // slot index: every row walks its rungs 16, 8, 4, 2, centroid — the costliest items first, the
    // cheapest in the tail.  (Letting odd rows walk 4, 2, 16, 8, centroid, so that some SMs stream wide
    // blocks while others unpack narrow ones, measured 12 % slower on the 16k-token workload.)
    // the row's six class starts in two loads (the table rows are 32 bytes, aligned): one round trip per
    // drawn item instead of one per class walked
    const int4 t0 = *reinterpret_cast<const int4*>(tab);
    const int2 t1 = *reinterpret_cast<const int2*>(tab + 4);
    const int st[6] = {t0.x, t0.y, t0.z, t0.w, t1.x, t1.y};
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        const int start = st[k], cnt = st[k + 1] - start;
        const int ck = k == 4 ? min(p.chunk, kMaxCentroidItemBlocks) : p.chunk;
        const int n = (cnt + ck - 1) / ck;
        if (slot < n) {
            sp.level = ladder_level(k);
            sp.b_lo = start + slot * ck;
            sp.nblk = min(ck, cnt - slot * ck);
            return sp;
        }
        slot -= n;
    }
    return sp;
}

struct ProducerState {
    uint32_t head = 0, used = 0;
    int seq_alloc = 0, seq_free = 0;
};

// One stream's blocks of one item.  Ring bookkeeping is done by all lanes alike (same values
// everywhere, so nothing has to be broadcast); lane 0 publishes the slot descriptor and starts ONE
// bulk copy for the block's bytes; the four scale planes of a quantised rung are fetched by all 32
// lanes with 16-byte asynchronous copies that arrive on the same barrier.
// Non-blocking test of a barrier phase.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}

// One stream's blocks of one item, in BATCHES: the warp reclaims the slots the consumers have
// finished, works out (all lanes alike, plain integer arithmetic) how many of the item's next blocks
// fit into the ring right now and where, and then lane i takes block i of the batch: it publishes the
// slot descriptor, arms the slot's barrier and starts ONE bulk copy for the block's bytes.  The four
// scale planes of a quantised rung are then fetched block by block by all 32 lanes with 16-byte
// asynchronous copies that arrive on the same barrier.  A producer that handles one block per loop
// iteration is bound by the latency of its own chain of ~60 dependent instructions (~1300 cycles per
// block measured); batches overlap those chains, and a producer that has fallen behind catches up.
template <int D, int G>
__device__ __forceinline__ bool produce_item(const Params& p, const TensorMaps& tm, Smem<D, G>& sm, ProducerState& ps, int s,
                                             const ItemDesc& it, int islot) {
    using C = Cfg<D, G>;
    const int lane = threadIdx.x & 31;
    if (it.level == 1 || it.nblk == 0) return true;     // centroid items are read straight from global memory
    const int j0 = (s ^ it.first) & 1;                   // this stream's first block of the item
    const int n_mine = (it.nblk - j0 + 1) >> 1;
    const uint32_t tab = smem_u32(sm.item_tab + islot * kMaxItemBlocks + j0);      // this stream's blocks: every second entry
    const int lv = it.level;
    const bool quant = lv != 16;
    const uint32_t dbytes = 2u * (uint32_t)half_bytes(lv, D);
    constexpr int K = C::KSCALE;                         // == VSCALE: every scale plane has the same bytes per block
    static_assert(C::KSCALE == C::VSCALE && (4 * K) % 512 == 0, "scale planes");
    constexpr int NR = 4 * K / 512;                      // rounds of 32 lanes x 16 bytes that cover the four planes
    const uint32_t need = (dbytes + (quant ? 4u * K : 0u) + 1023u) & ~1023u;
    // tiled copies: the tile row width of the item's rung (0: plain bulk copy) and its tensor map
    const int tw = lv == 16 ? Lay<D, G, 16>::W : lv == 8 ? Lay<D, G, 8>::W : lv == 4 ? Lay<D, G, 4>::W : 0;
    const CUtensorMap* tmap = &tm.m[lv == 16 ? 0 : lv == 8 ? 1 : 2];
    // This lane's 16 bytes of every round: which plane, and where inside a block's K bytes — fixed for the item.
    const uint8_t* splane[NR];
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int o = i * 512 + lane * 16, which = o / K;           // 0 klo, 1 kstep, 2 vlo, 3 vstep
        const uint8_t* base = reinterpret_cast<const uint8_t*>(which == 0 ? p.klo : which == 1 ? p.kstep
                                                               : which == 2 ? p.vlo : p.vstep);
        splane[i] = base + (size_t)it.row * p.nb * K + (o - which * K);
    }
    uint64_t* full = sm.full + s * kNSlot;
    uint64_t* empty = sm.empty + s * kNSlot;
    Desc* desc = sm.desc + s * kNSlot;
    const uint32_t ring = smem_u32(sm.ring) + (uint32_t)s * kRingBytes;
    for (int j = 0; j < n_mine;) {
        // slots the consumers are done with (oldest first; all lanes, same result everywhere)
        while (ps.seq_free < ps.seq_alloc) {
            const int sl = ps.seq_free % kNSlot;
            if (!mbar_test(&empty[sl], (uint32_t)(ps.seq_free / kNSlot) & 1u)) break;
            ps.used -= (uint32_t)desc[sl].pad;
            ++ps.seq_free;
        }
        // how many of the next blocks fit, and where this lane's block goes
        int nfit = 0;
        uint32_t my_dst = 0, my_pad = 0;
        {
            uint32_t head = ps.head, used = ps.used;
            const int slots = kNSlot - (ps.seq_alloc - ps.seq_free);
            const int want = min(min(n_mine - j, 32), slots);
            while (nfit < want) {
                const uint32_t waste = (head + need > kRingBytes) ? kRingBytes - head : 0u;
                if (used + waste + need > kRingBytes) break;
                const uint32_t dst = waste ? 0u : head;
                if (lane == nfit) { my_dst = dst; my_pad = waste + need; }
                used += waste + need;
                head = dst + need;
                if (head >= kRingBytes) head = 0;
                ++nfit;
            }
            if (nfit == 0) {                             // nothing fits: wait for the oldest block to be released
                const int sl = ps.seq_free % kNSlot;
                if (!mbar_wait(&empty[sl], (uint32_t)(ps.seq_free / kNSlot) & 1u)) return false;
                ps.used -= (uint32_t)desc[sl].pad;
                ++ps.seq_free;
                continue;
            }
            ps.head = head;
            ps.used = used;
        }
        const int my_seq = ps.seq_alloc + lane;
        const int my_slot = my_seq % kNSlot;
        uint4 cur = make_uint4(0, 0, 0, 0);
        bool withhold = false;
        if (lane < nfit) {
            cur = lds_v4(tab + 32u * (uint32_t)(j + lane));
#ifdef GKV_TEST_WITHHOLD_BLOCK
            // test build only: the second block of stream 0 never arrives, so the waits on it run out
            withhold = s == 0 && my_seq == 1;
#endif
            Desc d;
            d.off = my_dst; d.nvalid = (int)((cur.z >> 8) & 0xffu); d.pad = (int32_t)my_pad; d.orig = (int32_t)cur.w;
            desc[my_slot] = d;
            const unsigned long long soff = ((unsigned long long)cur.y << 32) | cur.x;      // byte offset in the cache
            const uint8_t* src = p.data + soff;
            if (withhold) {
            } else if (tw && tm.usable && (soff & (unsigned long long)(tw - 1)) == 0) {
                // a box of tile rows, written swizzled (row = byte offset / row width)
                mbar_arrive_tx(&full[my_slot], dbytes);
                tma_tile_g2s(ring + my_dst, tmap, 0, (int)(soff / (unsigned)tw), &full[my_slot]);
            } else if (!tw && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                mbar_arrive_tx(&full[my_slot], dbytes);
                bulk_g2s(ring + my_dst, src, dbytes, &full[my_slot]);
            } else {
                // block start not aligned for a bulk copy (a cache row at an odd address): this lane
                // copies the bytes by hand, into the layout the rung's consumers expect
                uint8_t* d0 = sm.ring + (size_t)s * kRingBytes + my_dst;
                if (tw == 128) for (uint32_t i = 0; i < dbytes; ++i) d0[swz<128>(i)] = src[i];
                else if (tw == 64) for (uint32_t i = 0; i < dbytes; ++i) d0[swz<64>(i)] = src[i];
                else if (tw == 32) for (uint32_t i = 0; i < dbytes; ++i) d0[swz<32>(i)] = src[i];
                else for (uint32_t i = 0; i < dbytes; ++i) d0[i] = src[i];
                __threadfence_block();
                mbar_arrive(&full[my_slot]);
            }
        }
        __syncwarp();
        // the four scale planes (a few hundred bytes each) of every block of the batch: 16 bytes per lane
        // and round, asynchronous, reporting to the block's barrier (one bulk copy per plane would cost
        // the warp ~200 cycles each)
        const unsigned held = __ballot_sync(0xffffffffu, withhold);
#pragma unroll 2
        for (int i = 0; i < nfit; ++i) {
            const uint32_t dst_i = __shfl_sync(0xffffffffu, my_dst, i);
            const uint32_t orig_i = __shfl_sync(0xffffffffu, cur.w, i);
            const int slot_i = (ps.seq_alloc + i) % kNSlot;
            if ((held >> i) & 1u) continue;
            if (quant) {
                const uint32_t sdst = ring + dst_i + dbytes + (uint32_t)lane * 16u;
                if (p.paged) {
                    // the planes follow the block's bytes in the pool, in the order the ring keeps them
                    const uint32_t ox = __shfl_sync(0xffffffffu, cur.x, i), oy = __shfl_sync(0xffffffffu, cur.y, i);
                    const uint8_t* sp = p.data + ((((unsigned long long)oy) << 32) | ox) + dbytes + (uint32_t)lane * 16u;
#pragma unroll
                    for (int r = 0; r < NR; ++r) cp_async16(sdst + (uint32_t)(r * 512), sp + r * 512);
                } else {
                    const size_t so = (size_t)orig_i * K;
#pragma unroll
                    for (int r = 0; r < NR; ++r) cp_async16(sdst + (uint32_t)(r * 512), splane[r] + so);
                }
            }
            cp_async_arrive(&full[slot_i]);              // one arrival per lane once its copies have landed
        }
        ps.seq_alloc += nfit;
        j += nfit;
    }
    return true;
}

// The scheduler warp draws the work items (an atomic counter), looks up what each one is, fetches
// its block entries into the item's table in shared memory and announces it — up to kItemSlots - 1
// items ahead of the consumers, so none of this global-memory latency is ever waited for by the
// producers or the consumers.  Items without blocks are not announced: their records are marked
// empty right here.
template <int D, int G>
__device__ void scheduler_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    const int lane = threadIdx.x & 31;
    int tot0 = 0, tot1 = 0, nfirst = 0;
    bool ok = true;
    for (int j = 0; ok; ++j) {
        ItemDesc it;
        for (;;) {                                          // draw the next item that has blocks
            int id = 0;
            if (lane == 0) id = atomicAdd(p.counter, 1);
            id = __shfl_sync(0xffffffffu, id, 0);
            const Span sp = span_of(p, id);                 // same loads in every lane (broadcast)
            it.item = id; it.row = sp.row; it.level = sp.level; it.b_lo = sp.b_lo; it.nblk = sp.nblk;
            it.exit = id >= p.items ? 1 : 0;
            it.pad[0] = it.pad[1] = it.pad[2] = 0;
            if (it.exit || sp.nblk > 0) break;
            // an empty slot of the row: nothing to do and nothing to write — the used slots of a row are a
            // prefix of its slots, and the merge kernel works out from the row's class counts how many
            // there are, so it never reads the records of an empty slot
        }
        it.first = nfirst & 1;
        if (!it.exit && it.level != 1) {
            const int n0 = (it.nblk + 1) >> 1, n1 = it.nblk >> 1;       // the first stream gets the odd block
            if (it.first) { tot1 += n0; tot0 += n1; } else { tot0 += n0; tot1 += n1; }
            ++nfirst;
        }
        it.end_seq0 = tot0;
        it.end_seq1 = tot1;
        // the item's block entries, four per lane, with the row's base offset added
        constexpr int kPerLane = kMaxItemBlocks / 32;
        uint4 e[kPerLane];
#pragma unroll
        for (int h = 0; h < kPerLane; ++h) {
            e[h] = make_uint4(0, 0, 0, 0);
            const int i = lane + 32 * h;
            if (!it.exit && i < it.nblk) {
                e[h] = p.plan[(size_t)(p.per_row_meta ? it.row : 0) * p.nb + it.b_lo + i];
                const unsigned long long src = (unsigned long long)it.row * (unsigned long long)p.stride_bh +
                                               (((unsigned long long)e[h].y << 32) | e[h].x);
                e[h].x = (uint32_t)src; e[h].y = (uint32_t)(src >> 32);
            }
        }
        // the descriptor slot is free once everybody has finished item j - kItemSlots
        const int sl = j % kItemSlots;
        if (j >= kItemSlots) ok = mbar_wait(&sm.item_empty[sl], (uint32_t)(j / kItemSlots - 1) & 1u);
        if (!ok) break;
#pragma unroll
        for (int h = 0; h < kPerLane; ++h) sm.item_tab[sl * kMaxItemBlocks + lane + 32 * h] = e[h];
        if (lane == 0) sm.item[sl] = it;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.item_full[sl]);
        if (it.exit) return;
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    }
    if (!ok && lane == 0) {
        atomicExch(p.status, 1);
        atomicExch(abort_flag, 1);
    }
}

// Producer of stream s: for every announced item, streams the item's blocks of its stream into its ring.
template <int D, int G>
__device__ void producer_loop(const Params& p, const TensorMaps& tm, Smem<D, G>& sm, int s, int* abort_flag) {
    const int lane = threadIdx.x & 31;
    ProducerState ps;
    bool ok = true;
    for (int j = 0; ok; ++j) {
        const int sl = j % kItemSlots;
        if (!mbar_wait(&sm.item_full[sl], (uint32_t)(j / kItemSlots) & 1u)) { ok = false; break; }
        const ItemDesc it = sm.item[sl];
        if (it.exit) return;
        ok = produce_item<D, G>(p, tm, sm, ps, s, it, sl);
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.item_empty[sl]);      // this warp no longer needs the item's descriptor and table
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    }
    if (!ok && lane == 0) {
        atomicExch(p.status, 9 + s);
        atomicExch(abort_flag, 1);
    }
}

// ================================ query warp ==================================================
// For every announced item: the row's query heads as fp32 (for the centroid path), a per-head
// power-of-two scale, and the MMA A-fragment planes (hi, lo) in the channel arrangement of the
// item's rung, into the buffer of the item's parity.  Runs one item ahead of the consumers.
template <int D, int G, bool DUP>
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
        // a centroid item needs the fp32 rows only (its blocks are not scored through the MMA planes)
        // per-head power-of-two scale bringing max|q| into [8, 16)
        for (int h = 0; h < 8 && it.level != 1; ++h) {
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
        // This lane writes its own fragment lane of every chunk: 8 halves (two k-steps x four slots)
        // per plane and chunk, as one 16-byte store.
        if (it.level != 1) {
            const int r = lane >> 2, t = lane & 3;
            const int head = head_of_row<DUP>(r);
            const float sc = sf[8 + head];
            const float* qr = sq + head * D + C::DT * t;
            const int bits = it.level;
#pragma unroll 1
            for (int i = 0; i < C::CH; ++i) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int jp = 0; jp < 4; ++jp) {            // halves 2jp, 2jp+1: k-step 2i + (jp >> 1), slots 2(jp & 1) + {0, 1}
                    const int ks = 2 * i + (jp >> 1), e0 = 2 * (jp & 1);
                    const float x0 = qr[arr_chan(bits, ks, e0)] * sc * arr_scale(bits, e0);
                    const float x1 = qr[arr_chan(bits, ks, e0 + 1)] * sc * arr_scale(bits, e0 + 1);
                    if (bits != 16) split_f16x2(x0, x1, hi[jp], lo[jp]);
                    else split_bf16x2(x0, x1, hi[jp], lo[jp]);
                }
                uint4* dst = reinterpret_cast<uint4*>(qp + ((size_t)i * 32 + lane) * 8);
                dst[0] = make_uint4(hi[0], lo[0], hi[1], lo[1]);                 // A registers a0..a3 of k-step 2i
                dst[C::QPLANE / 8] = make_uint4(hi[2], lo[2], hi[3], lo[3]);     // ... and of k-step 2i+1
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

// ================================ consumers ===================================================
// The blocks are processed in UNITS of G tokens (one token group of the K scales): scores of
// the unit, online-softmax update, value product of the unit.  All shared-memory operands are
// addressed by 32-bit shared addresses built from one per-thread base plus compile-time offsets.
template <int D, int G>
struct Unit {
    static constexpr int U = G;          // tokens
    static constexpr int NU = G / 8;     // token n-tiles
    static constexpr int KU = G / 16;    // PV k-steps
    static constexpr int ZN = G / 4;     // scores held per thread
};

template <int D, int G>
struct WarpState {
    using C = Cfg<D, G>;
    float o[C::MT][4];      // transposed output: channel rows (c0,c1) and their partners (c2,c3), head columns 2t, 2t+1; scaled 2^-16
    float ob[4];            // sum_j p_j * vlo[j][cg] for cg = r mod GV (c0, c1), head columns 2t, 2t+1; scaled 2^8
    float m;                // running reference of this thread's head (log2 domain), uniform over the quad
    float l;                // this thread's share of the running sum
};

template <int D, int G>
struct Ctx {                             // per-thread constants of the consumer role
    uint32_t qprep;                      // shared address of this lane's first prepared-query chunk (hi plane)
    uint32_t sq;                         // shared address of the fp32 query rows
    float f;                             // 2^-eq * log2(e) of this thread's head
    int r, t, lane;
    bool part;                           // with head pairs in the rows: this thread feeds the lo column of its head
};

template <int D, int G>
__device__ __forceinline__ uint4 qchunk(const Ctx<D, G>& c, int plane, int i) {
    return lds_v4(c.qprep + (uint32_t)(plane * Cfg<D, G>::QPLANE * 2 + i * 512));
}

// ---- K side of one unit of a quantised block: scores in the log2 domain ---------------------------
// Score column n of n-tile j stands for token 8j + n of the unit.
template <int D, int G, int BITS>
__device__ __forceinline__ void scores_unit(const Ctx<D, G>& c, uint32_t blk, int tg, float (&z)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr int RB = D * BITS / 8;                     // bytes per token row
    constexpr int TB = RB / 4;                           // bytes per thread per row
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
    // every fetch stays inside one 16-byte chunk, so in a swizzled block only the chunk moves (rows 8n + r of
    // all n-tiles have the same XOR term)
    static_assert(LB <= 16, "a fetch must not cross a 16-byte chunk");
    const uint32_t kx = swz_term<D, G, BITS>(c.r, 0);
    const uint32_t rowbase = blk + (uint32_t)((tg * UU::U + c.r) * RB);

    float acc[UU::NU][4];                                // first written by the MMAs of chunk 0 (accumulator input zero)
    // q . klo of this token group rides along as one more n-tile whose eight columns all carry the
    // group's klo (so every thread ends up with its own head's value, no shuffle); two accumulators,
    // one per k-step of a chunk, keep the MMAs independent.
    float bias0[4], bias1[4];
#pragma unroll
    for (int g = 0; g < C::CH / CG; ++g) {
        uint32_t W[UU::NU][LW];
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) {
            const uint32_t src = rowbase + (((uint32_t)(c.t * TB + g * LB)) ^ kx) + (uint32_t)(n * 8 * RB);
            if (LW == 4) { const uint4 v = lds_v4(src); W[n][0] = v.x; W[n][1 % LW] = v.y; W[n][2 % LW] = v.z; W[n][3 % LW] = v.w; }
            else if (LW == 2) { const uint2 v = lds_v2(src); W[n][0] = v.x; W[n][1 % LW] = v.y; }
            else W[n][0] = lds_u32(src);
        }
#pragma unroll
        for (int ii = 0; ii < CG; ++ii) {                // two k-steps at a time
            const int i = g * CG + ii;
            const uint4 qa = qchunk(c, 0, i), qb = qchunk(c, 1, i);      // (hi, lo, hi, lo) of k-steps 2i and 2i+1
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
            if (i == 0) {
                mma_f16_z(bias0, qa.x, qa.y, qa.z, qa.w, lp[0], lp[1]);
                mma_f16_z(bias1, qb.x, qb.y, qb.z, qb.w, lp[2], lp[3]);
            } else {
                mma_f16(bias0, qa.x, qa.y, qa.z, qa.w, lp[0], lp[1]);
                mma_f16(bias1, qb.x, qb.y, qb.z, qb.w, lp[2], lp[3]);
            }
            uint32_t a[8];
            mul_split(qa.x, qa.y, sp[0], a[0], a[1]);
            mul_split(qa.z, qa.w, sp[1], a[2], a[3]);
            mul_split(qb.x, qb.y, sp[2], a[4], a[5]);
            mul_split(qb.z, qb.w, sp[3], a[6], a[7]);
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
            for (int n = 0; n < UU::NU; ++n) {
                if (i == 0) mma_f16_z(acc[n], a[0], a[1], a[2], a[3], bb[n][0], bb[n][1]);
                else mma_f16(acc[n], a[0], a[1], a[2], a[3], bb[n][0], bb[n][1]);
            }
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
    // swizzled block: this thread's 16-byte chunks of a row all share the row's XOR term
    const uint32_t bt = (uint32_t)(C::DT * c.t * 2);
    const uint32_t kx = swz_term<D, G, 16>(c.r, (int)bt);
    const uint32_t rowbase = blk + (uint32_t)((tg * UU::U + c.r) * D * 2);
    float acc[UU::NU][4];
#pragma unroll
    for (int i = 0; i < C::CH; ++i) {
        const uint4 qa = qchunk(c, 0, i), qb = qchunk(c, 1, i);
        uint4 w[UU::NU];
        const uint32_t coff = (bt + 16u * (uint32_t)i) ^ kx;
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) w[n] = lds_v4(rowbase + coff + n * 8 * D * 2);
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) {
            if (i == 0) mma_bf16_z(acc[n], qa.x, qa.y, qa.z, qa.w, w[n].x, w[n].y);
            else mma_bf16(acc[n], qa.x, qa.y, qa.z, qa.w, w[n].x, w[n].y);
        }
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) mma_bf16(acc[n], qb.x, qb.y, qb.z, qb.w, w[n].z, w[n].w);
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
// the accumulator rescale off the common path; the fp16 weight operands still fit
// (p * 2^8 * step < 65504 for any step < 16).
constexpr float kLazy = 4.0f;

// The accumulators are indexed by head COLUMN (2t, 2t+1) while the reference belongs to the head of
// the thread's ROW, so the rescale factors of the two columns come from the lanes that own them.
template <int D, int G, bool DUP>
__device__ __forceinline__ float move_reference(const Ctx<D, G>& c, WarpState<D, G>& st, float mx) {
    using C = Cfg<D, G>;
    const bool need = mx > st.m + kLazy || st.m == -INFINITY;   // per head (uniform over the quad)
    if (__any_sync(0xffffffffu, need)) {
        const float mnew = need ? mx : st.m;
        const float corr = ex2(st.m - mnew);          // 0 when st.m = -inf, 1 for the heads that stay
        st.m = mnew;
        st.l *= corr;
        // column 2t is head t (and 2t+1 its lo column), or heads 2t and 2t+1; row 2h (resp. h) is a thread of head h
        const float c0 = __shfl_sync(0xffffffffu, corr, 8 * c.t);
        const float c1 = DUP ? c0 : __shfl_sync(0xffffffffu, corr, 8 * c.t + 4);
#pragma unroll
        for (int n = 0; n < C::MT; ++n) {
            st.o[n][0] *= c0; st.o[n][1] *= c1; st.o[n][2] *= c0; st.o[n][3] *= c1;
        }
        st.ob[0] *= c0; st.ob[1] *= c1; st.ob[2] *= c0; st.ob[3] *= c1;
    }
    return st.m;
}

// z: scores of this thread's head for the unit's tokens 8*n + 2t + {0,1} (log2 domain); nrel = valid
// tokens left in this unit (>= 1).  Returns the weights in z.
template <int D, int G, bool DUP>
__device__ __forceinline__ float softmax_unit(const Ctx<D, G>& c, WarpState<D, G>& st, float (&z)[Unit<D, G>::ZN], int nrel) {
    using UU = Unit<D, G>;
    float mx = -INFINITY;
    if (nrel >= UU::U) {                                 // full unit (the common case): no masks
#pragma unroll
        for (int i = 0; i < UU::ZN; ++i) mx = fmaxf(mx, z[i]);
    } else {
#pragma unroll
        for (int i = 0; i < UU::ZN; ++i) {
            const int tok = (i >> 1) * 8 + 2 * c.t + (i & 1);
            if (tok >= nrel) z[i] = -INFINITY;
            mx = fmaxf(mx, z[i]);
        }
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m = move_reference<D, G, DUP>(c, st, mx);
    float ls = 0.f;
#pragma unroll
    for (int i = 0; i < UU::ZN; ++i) {
        z[i] = ex2(z[i] - m);
        ls += z[i];
    }
    st.l += ls;
    return ls;                                           // this thread's share of the unit's weights (reference st.m)
}

// Pairs (x[tok][cg], x[tok+1][cg]) of a (64, GV) fp16 plane at shared address `row` (token `tok`, even).
template <int GV>
__device__ __forceinline__ void scale_pairs(uint32_t row, uint32_t (&out)[GV]) {
    if (GV == 8) {
        const uint4 a = lds_v4(row), b = lds_v4(row + 16);
        out[0] = prmt(a.x, b.x, 0x5410); out[1 % GV] = prmt(a.x, b.x, 0x7632);
        out[2 % GV] = prmt(a.y, b.y, 0x5410); out[3 % GV] = prmt(a.y, b.y, 0x7632);
        out[4 % GV] = prmt(a.z, b.z, 0x5410); out[5 % GV] = prmt(a.z, b.z, 0x7632);
        out[6 % GV] = prmt(a.w, b.w, 0x5410); out[7 % GV] = prmt(a.w, b.w, 0x7632);
    } else if (GV == 4) {
        const uint4 v = lds_v4(row);
        out[0] = prmt(v.x, v.z, 0x5410); out[1 % GV] = prmt(v.x, v.z, 0x7632);
        out[2 % GV] = prmt(v.y, v.w, 0x5410); out[3 % GV] = prmt(v.y, v.w, 0x7632);
    } else if (GV == 2) {
        const uint2 v = lds_v2(row);
        out[0] = prmt(v.x, v.y, 0x5410); out[1 % GV] = prmt(v.x, v.y, 0x7632);
    } else {
#pragma unroll
        for (int cg = 0; cg < GV; ++cg) out[cg] = lds_u16(row + 2 * cg) | (lds_u16(row + 2 * GV + 2 * cg) << 16);
    }
}

// ---- V side: the transposed product O^T[channel][head] += V^T[channel][token] * (p*vstep)[token][head] -------
// How a thread's value codes reach its A registers.  A SPAN is the set of channels whose codes one
// fetch delivers: the 16-byte chunk of a token row that ldmatrix.trans hands out (128/BITS channels;
// used for 8-bit codes, and for 4-bit codes when a channel group is at least a chunk), or one
// channel group fetched with a plain byte load (2-bit codes, and 4-bit codes with 16-channel groups).
// Either way thread r owns F = SP/8 neighbouring fields of every span, fields 2k and 2k+1 feed rows r
// and r+8 of the span's m-tile k, and the register R = {fields of token a | fields of token a+1 << 16}
// is unpacked by one shift and two masks per m-tile: the even field lands on bit POS, the odd one
// BITS higher, so rows r+8 carry 2^BITS more weight, which the epilogue takes back out.
template <int D, int G, int BITS>
struct VT {
    static constexpr bool LDSM = BITS == 8 || (BITS == 4 && G >= 32);
    static constexpr int SP = LDSM ? 128 / BITS : G;     // channels per span
    static constexpr int F = SP / 8;                     // fields per thread and span
    static constexpr int MTS = F / 2;                    // m-tiles per span
    static constexpr int SPC = G / SP;                   // spans per channel group
    static constexpr int NSPAN = D / SP;
    static constexpr int RB = D * BITS / 8;
    static constexpr int POS = BITS == 4 ? 3 : BITS == 2 ? 6 : 0;
    static constexpr int LOAD_BITS = F * BITS;           // bits of one token a thread needs per span (plain-load path)
    static_assert(F >= 2 && F % 2 == 0 && SPC >= 1, "unsupported shape");
};
__host__ __device__ constexpr float v_pscale(int bits) { return bits == 4 ? 32.f : bits == 2 ? 4.f : 256.f; }   // 2^(8-POS)
__host__ __device__ constexpr float v_rowscale(int bits) { return bits == 4 ? 16.f : bits == 2 ? 4.f : 1.f; }   // weight of rows r+8 over rows r

// A registers (rows r, r+8) of m-tile k of a span from R (the thread's first field at bit 0 of each half).
template <int BITS, int POS>
__device__ __forceinline__ void extract_pair(uint32_t R, int k, uint32_t& even, uint32_t& odd) {
    if (BITS == 8) {
        even = prmt(R, 0u, 0x4240);
        odd = prmt(R, 0u, 0x4341);
    } else {
        constexpr uint32_t FM = (1u << BITS) - 1u;
        const int sh = POS - 2 * k * BITS;
        const uint32_t u = sh >= 0 ? (R << sh) : (R >> (-sh));
        even = u & ((FM << POS) * 0x00010001u);
        odd = u & ((FM << (POS + BITS)) * 0x00010001u);
    }
}

// Part of (ph + pl) * s that this thread's column carries: hi = rn(ph*s) or lo = rn(pl*s + (ph*s - hi)).
__device__ __forceinline__ uint32_t mul_part(uint32_t ph, uint32_t pl, uint32_t s, bool lo_part) {
    const __half2 h = __hmul2(u32_as_h2(ph), u32_as_h2(s));
    const __half2 e = __hfma2(u32_as_h2(ph), u32_as_h2(s), __hneg2(h));
    const __half2 l = __hfma2(u32_as_h2(pl), u32_as_h2(s), e);
    return lo_part ? h2_as_u32(l) : h2_as_u32(h);
}

template <int D, int G, int BITS, bool DUP>
__device__ __forceinline__ void values_unit(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int unit,
                                            const float (&pz)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    using V = VT<D, G, BITS>;
    constexpr int RB = V::RB;
    constexpr float PSCALE = v_pscale(BITS);
    const uint32_t vbase = blk + (uint32_t)(kP * RB);
    const uint32_t sbase = blk + (uint32_t)(2 * (kP * RB) + 2 * C::KSCALE);       // vlo plane; vstep follows
    const int tok0 = unit * UU::U + 2 * c.t;            // lower token of this thread's first pair
    // ldmatrix row of this lane: token (lane & 7) of the first or second half of a k-step, chunk +0 / +1; in a
    // swizzled block the chunk index is XORed with the row's term (the same for every row this lane addresses)
    const uint32_t vx = swz_term<D, G, BITS>(c.lane & 7, 0);
    const uint32_t ldsm_lane = vbase + (uint32_t)((unit * UU::U + (c.lane & 7) + 8 * ((c.lane >> 3) & 1)) * RB) +
                               ((uint32_t)(16 * (c.lane >> 4)) ^ (vx & 16u));
    const uint32_t vxe = vx & ~16u;
    // plain-load path: this thread's fields of (token tok0, span 0)
    const uint32_t lds_lane = vbase + (uint32_t)(tok0 * RB + (c.r * V::LOAD_BITS) / 8);
    const int sub = (V::LOAD_BITS % 8) ? ((c.r * V::LOAD_BITS) & 7) : 0;
    const int cgr = c.r % C::GV;
#pragma unroll
    for (int ku = 0; ku < UU::KU; ++ku) {
        uint32_t ph[2], pl[2];
        split_f16x2(pz[4 * ku + 0] * PSCALE, pz[4 * ku + 1] * PSCALE, ph[0], pl[0]);
        split_f16x2(pz[4 * ku + 2] * PSCALE, pz[4 * ku + 3] * PSCALE, ph[1], pl[1]);
        const uint32_t srow = sbase + (uint32_t)((tok0 + 16 * ku) * C::GV * 2);
        uint32_t sa[C::GV], sb[C::GV];
        scale_pairs<C::GV>(srow + C::VSCALE, sa);                      // vstep of the pair in n-tile 2ku
        scale_pairs<C::GV>(srow + C::VSCALE + 8 * C::GV * 2, sb);      // ... and of the pair in n-tile 2ku+1
        // p . vlo: row r of this tile is channel group r mod GV
        {
            uint32_t la = lds_u16(srow + 2 * cgr) | (lds_u16(srow + 2 * C::GV + 2 * cgr) << 16);
            uint32_t lb = lds_u16(srow + 16 * C::GV + 2 * cgr) | (lds_u16(srow + 18 * C::GV + 2 * cgr) << 16);
            if (V::POS) {                               // keep the 2^8 scale of the p . vlo accumulator
                const __half2 lo_scale = __float2half2_rn((float)(1 << V::POS));
                la = h2_as_u32(__hmul2(u32_as_h2(la), lo_scale));
                lb = h2_as_u32(__hmul2(u32_as_h2(lb), lo_scale));
            }
            if (DUP) {
                mma_f16(st.ob, la, 0u, lb, 0u, c.part ? pl[0] : ph[0], c.part ? pl[1] : ph[1]);
            } else {
                mma_f16(st.ob, la, 0u, lb, 0u, ph[0], ph[1]);
                mma_f16(st.ob, la, 0u, lb, 0u, pl[0], pl[1]);
            }
        }
        // value codes of this k-step: Rlo[s] / Rhi[s] = span s, token pairs of n-tiles 2ku / 2ku+1
        uint32_t Rlo[V::NSPAN], Rhi[V::NSPAN];
        if (V::LDSM) {
#pragma unroll
            for (int s2 = 0; s2 < V::NSPAN / 2; ++s2)
                ldsm_x4_trans(ldsm_lane + (uint32_t)(ku * 16 * RB) + ((uint32_t)(32 * s2) ^ vxe), Rlo[2 * s2], Rhi[2 * s2],
                              Rlo[(2 * s2 + 1) % V::NSPAN], Rhi[(2 * s2 + 1) % V::NSPAN]);
        } else {
#pragma unroll
            for (int s = 0; s < V::NSPAN; ++s) {
                uint32_t x[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t src = lds_lane + (uint32_t)((16 * ku + ((k & 2) ? 8 : 0) + (k & 1)) * RB + (s * V::SP * BITS) / 8);
                    x[k] = V::LOAD_BITS > 8 ? lds_u16(src) : (lds_u8(src) >> sub);
                }
                Rlo[s] = prmt(x[0], x[1], 0x5410);
                Rhi[s] = prmt(x[2], x[3], 0x5410);
            }
        }
#pragma unroll
        for (int cg = 0; cg < C::GV; ++cg) {
            uint32_t b0h, b0l, b1h, b1l;
            if (DUP) {
                b0h = mul_part(ph[0], pl[0], sa[cg], c.part);
                b1h = mul_part(ph[1], pl[1], sb[cg], c.part);
                b0l = b1l = 0u;
            } else {
                mul_split(ph[0], pl[0], sa[cg], b0h, b0l);
                mul_split(ph[1], pl[1], sb[cg], b1h, b1l);
            }
#pragma unroll
            for (int sc = 0; sc < V::SPC; ++sc) {
                const int s = cg * V::SPC + sc;
#pragma unroll
                for (int k = 0; k < V::MTS; ++k) {
                    uint32_t a0, a1, a2, a3;
                    extract_pair<BITS, V::POS>(Rlo[s], k, a0, a1);
                    extract_pair<BITS, V::POS>(Rhi[s], k, a2, a3);
                    float (&acc)[4] = st.o[s * V::MTS + k];
                    mma_f16(acc, a0, a1, a2, a3, b0h, b1h);
                    if (!DUP) mma_f16(acc, a0, a1, a2, a3, b0l, b1l);
                }
            }
        }
    }
}

// Raw bf16 values: m-tile m is channels 16m .. 16m+15 in natural order; ldmatrix.trans delivers the
// four A registers of a (k-step, m-tile) directly.
template <int D, int G, bool DUP>
__device__ __forceinline__ void values_unit_bf16(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int unit,
                                                 const float (&pz)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr float kScale = 1.52587890625e-05f;      // 2^-16: same accumulator scale as the code path
    constexpr int RB = D * 2;
    // matrices: (tokens of n-tile 2ku, channels 16m..), (same tokens, 16m+8..), (n-tile 2ku+1, 16m..), (n-tile 2ku+1, 16m+8..)
    // swizzled: chunk (2m + b) of a row, b = (lane >> 3) & 1, is XORed with the term of its 128-byte tile row
    const uint32_t rowb = blk + (uint32_t)(kP * RB + (unit * UU::U + (c.lane & 7) + 8 * (c.lane >> 4)) * RB);
    const uint32_t cb = 16u * ((c.lane >> 3) & 1);
    const uint32_t vx0 = swz_term<D, G, 16>(c.lane & 7, 0), vx1 = swz_term<D, G, 16>(c.lane & 7, 128);   // first / second 128 bytes of the row
#pragma unroll
    for (int ku = 0; ku < UU::KU; ++ku) {
        uint32_t ph[2], pl[2];
        split_bf16x2(pz[4 * ku + 0] * kScale, pz[4 * ku + 1] * kScale, ph[0], pl[0]);
        split_bf16x2(pz[4 * ku + 2] * kScale, pz[4 * ku + 3] * kScale, ph[1], pl[1]);
        const uint32_t b0 = DUP ? (c.part ? pl[0] : ph[0]) : ph[0];
        const uint32_t b1 = DUP ? (c.part ? pl[1] : ph[1]) : ph[1];
#pragma unroll
        for (int m = 0; m < C::MT; ++m) {
            uint32_t a0, a1, a2, a3;
            const uint32_t off = (uint32_t)(32 * m) + cb;                 // byte of the chunk inside the row
            const uint32_t phys = (32 * m >= 128) ? (off ^ vx1) : (off ^ vx0);
            ldsm_x4_trans(rowb + (uint32_t)(ku * 16 * RB) + phys, a0, a1, a2, a3);
            mma_bf16(st.o[m], a0, a1, a2, a3, b0, b1);
            if (!DUP) mma_bf16(st.o[m], a0, a1, a2, a3, pl[0], pl[1]);
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

// Channel of row r (odd = 0) or r+8 (odd = 1) of output m-tile mt, for each rung's value layout.
template <int D, int G, int BITS>
__device__ __forceinline__ int out_channel(int mt, int r, int odd) {
    if (BITS == 16) return 16 * mt + r + 8 * odd;
    using V = VT<D, G, BITS == 16 ? 8 : BITS>;
    return V::SP * (mt / V::MTS) + V::F * r + 2 * (mt % V::MTS) + odd;
}

// This warp's record of an item (natural-log domain): m, l, o[D] per head.
template <int D, int G, int BITS, bool DUP>
__device__ __forceinline__ void write_record(const Params& p, const Ctx<D, G>& c, const WarpState<D, G>& st, float* rec0) {
    using C = Cfg<D, G>;
    float l = st.l;
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    const int myhead = head_of_row<DUP>(c.r);
    if (c.t == 0 && myhead < p.rep && (!DUP || (c.r & 1) == 0)) {
        float* rec = rec0 + (size_t)myhead * (D + 2);
        rec[0] = st.m * 0.6931471805599453f;
        rec[1] = l;
    }
    // p . vlo of channel group cg and column n sits in the lane of row cg, quad position n / 2, scaled 2^8
    const float ob0 = DUP ? st.ob[0] + st.ob[1] : st.ob[0], ob1 = st.ob[1];
    constexpr float kRow = 65536.f, kRow8 = 65536.f / v_rowscale(BITS);
#pragma unroll
    for (int mt = 0; mt < C::MT; ++mt) {
        const int ch0 = out_channel<D, G, BITS>(mt, c.r, 0), ch1 = out_channel<D, G, BITS>(mt, c.r, 1);
        float bias00 = 0.f, bias01 = 0.f, bias10 = 0.f, bias11 = 0.f;      // [channel row][column]
        if (BITS != 16) {
            const int l0 = ((ch0 / G) % 8) * 4 + c.t, l1 = ((ch1 / G) % 8) * 4 + c.t;
            bias00 = __shfl_sync(0xffffffffu, ob0, l0) * 0.00390625f;
            bias10 = __shfl_sync(0xffffffffu, ob0, l1) * 0.00390625f;
            if (!DUP) {
                bias01 = __shfl_sync(0xffffffffu, ob1, l0) * 0.00390625f;
                bias11 = __shfl_sync(0xffffffffu, ob1, l1) * 0.00390625f;
            }
        }
        if (DUP) {
            if (c.t < p.rep) {
                float* rec = rec0 + (size_t)c.t * (D + 2) + 2;
                rec[ch0] = fmaf(st.o[mt][0] + st.o[mt][1], kRow, bias00);
                rec[ch1] = fmaf(st.o[mt][2] + st.o[mt][3], kRow8, bias10);
            }
        } else {
            if (2 * c.t < p.rep) {
                float* rec = rec0 + (size_t)(2 * c.t) * (D + 2) + 2;
                rec[ch0] = fmaf(st.o[mt][0], kRow, bias00);
                rec[ch1] = fmaf(st.o[mt][2], kRow8, bias10);
            }
            if (2 * c.t + 1 < p.rep) {
                float* rec = rec0 + (size_t)(2 * c.t + 1) * (D + 2) + 2;
                rec[ch0] = fmaf(st.o[mt][1], kRow, bias01);
                rec[ch1] = fmaf(st.o[mt][3], kRow8, bias11);
            }
        }
    }
}

// One thread per head and unit reports the head's share of a block's softmax mass: the reference in use
// (natural-log domain) and the sum of the unit's weights against it.
template <int D, int G, bool DUP>
__device__ __forceinline__ void report_mass(const Params& p, const Ctx<D, G>& c, int row, int orig, int upb, int unit, float ref, float sum) {
    const int head = head_of_row<DUP>(c.r);
    if (c.t == 0 && head < p.rep && (!DUP || (c.r & 1) == 0))
        p.mass_part[(((size_t)row * p.nb + orig) * upb + unit) * p.rep + head] = make_float2(ref, sum);
}

// An item of one of the byte-ring rungs: this warp's blocks of its stream, then its record.
template <int D, int G, int BITS, bool DUP, bool MASS>
__device__ __forceinline__ int ring_item(
                                         const Params& p, Smem<D, G>& sm, const Ctx<D, G>& c, const ItemDesc& it,
                                      int stream, int u0, int u1, int& seq, float* rec0) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    WarpState<D, G> st;
#pragma unroll
    for (int n = 0; n < C::MT; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;
    st.ob[0] = st.ob[1] = st.ob[2] = st.ob[3] = 0.f;
    st.m = -INFINITY;
    st.l = 0.f;
    const uint32_t ring = smem_u32(sm.ring) + (uint32_t)stream * kRingBytes;
    uint64_t* full = sm.full + stream * kNSlot;
    uint64_t* empty = sm.empty + stream * kNSlot;
    const Desc* desc = sm.desc + stream * kNSlot;
    const int end = stream ? it.end_seq1 : it.end_seq0;
    for (; seq < end; seq += kPairsPerStream) {
        const int slot = seq % kNSlot;
        if (!mbar_wait(&full[slot], (uint32_t)(seq / kNSlot) & 1u)) return 4;
        const uint32_t off = desc[slot].off;
        const int nvalid = desc[slot].nvalid;
        const int orig = MASS ? desc[slot].orig : 0;
        const uint32_t blk = ring + off;
        // both warps of the pair clear the tail (same zeros, so the overlap is harmless)
        if (nvalid < kP) clear_invalid_tail<D, G>(sm.ring + (size_t)stream * kRingBytes + off, BITS, nvalid, c.lane);
        constexpr int UPB = kP / UU::U;
#pragma unroll 1
        for (int unit = u0; unit < u1; ++unit) {
            const int nrel = nvalid - unit * UU::U;
            if (nrel <= 0) {                             // no valid token in this unit: it weighs nothing
                if (MASS) report_mass<D, G, DUP>(p, c, it.row, orig, UPB, unit, -INFINITY, 0.f);
                if (MASS) continue;
                break;
            }
            float z[UU::ZN];
            if (BITS == 16) scores_unit_bf16<D, G>(c, blk, unit, z);
            else scores_unit<D, G, BITS == 16 ? 8 : BITS>(c, blk, unit, z);
            float ls = softmax_unit<D, G, DUP>(c, st, z, nrel);
            if (MASS) {
                ls += __shfl_xor_sync(0xffffffffu, ls, 1);
                ls += __shfl_xor_sync(0xffffffffu, ls, 2);
                report_mass<D, G, DUP>(p, c, it.row, orig, UPB, unit, st.m * 0.6931471805599453f, ls);
            }
            if (BITS == 16) values_unit_bf16<D, G, DUP>(c, st, blk, unit, z);
            else values_unit<D, G, BITS == 16 ? 8 : BITS, DUP>(c, st, blk, unit, z);
        }
        __syncwarp();
        if (c.lane == 0) mbar_arrive(&empty[slot]);
    }
    write_record<D, G, BITS, DUP>(p, c, st, rec0);
    return 0;
}

// An item of centroid blocks (one key and one value vector stand for nvalid tokens; 512 bytes per
// block at D = 128).  No ring: warp w takes blocks w, w + 12, ... of the item and reads each with one
// 16-byte load per lane straight from global memory — all of its loads are in flight before the first
// is used.  Lanes 0-15 own heads 0-3 and lanes 16-31 heads 4-7; lane l of a half owns channels
// 8(l & 15) .. +7 of the key (for the scores, reduced over the half) and of the value.
template <int D, int G, bool MASS>
__device__ __forceinline__ void centroid_item(const Params& p, const Ctx<D, G>& c, const ItemDesc& it, const uint4* tab,
                                              int warp, float* rec0) {
    constexpr int kMaxMine = (kMaxCentroidItemBlocks + kConsumerWarps - 1) / kConsumerWarps;
    constexpr int LPV = D / 8;                            // lanes that cover one vector with 16 bytes each
    static_assert(LPV <= 16, "head dim too large for the centroid path");
    const int lane = c.lane, hl = lane & 15, h0 = (lane >> 4) * 4;
    // this warp's blocks are entries warp, warp + 12, ... of the item's table (shared memory)
    const int nmine = it.nblk > warp ? (it.nblk - warp + kConsumerWarps - 1) / kConsumerWarps : 0;
    uint4 kraw[kMaxMine], vraw[kMaxMine];
    int nval[kMaxMine];
#pragma unroll
    for (int j = 0; j < kMaxMine; ++j) {
        nval[j] = 0;
        kraw[j] = vraw[j] = make_uint4(0, 0, 0, 0);
        if (j < nmine) {
            const uint4 e = tab[warp + kConsumerWarps * j];
            nval[j] = (int)((e.z >> 8) & 0xffu);
        }
        if (j < nmine && hl < LPV) {
            const uint4 e = tab[warp + kConsumerWarps * j];
            const uint8_t* src = p.data + (((unsigned long long)e.y << 32) | e.x);
            if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                kraw[j] = __ldg(reinterpret_cast<const uint4*>(src) + hl);
                vraw[j] = __ldg(reinterpret_cast<const uint4*>(src + 2 * D) + hl);
            } else {                                      // a cache row at an odd address: byte loads
                uint32_t w[8];
                for (int i = 0; i < 8; ++i) {
                    const uint8_t* s4 = src + (i < 4 ? 0 : 2 * D) + 16 * hl + 4 * (i & 3);
                    w[i] = (uint32_t)s4[0] | ((uint32_t)s4[1] << 8) | ((uint32_t)s4[2] << 16) | ((uint32_t)s4[3] << 24);
                }
                kraw[j] = make_uint4(w[0], w[1], w[2], w[3]);
                vraw[j] = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
    }
    // this lane's slice of its four heads' queries (fp32 rows prepared by the query warp)
    float q[4][8];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        const uint4 a = lds_v4(c.sq + (uint32_t)(((h0 + h) * D + 8 * (hl % LPV)) * 4));
        const uint4 b = lds_v4(c.sq + (uint32_t)(((h0 + h) * D + 8 * (hl % LPV) + 4) * 4));
        q[h][0] = __uint_as_float(a.x); q[h][1] = __uint_as_float(a.y); q[h][2] = __uint_as_float(a.z); q[h][3] = __uint_as_float(a.w);
        q[h][4] = __uint_as_float(b.x); q[h][5] = __uint_as_float(b.y); q[h][6] = __uint_as_float(b.z); q[h][7] = __uint_as_float(b.w);
    }
    float m[4], l[4], o[4][8];
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        m[h] = -INFINITY; l[h] = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[h][i] = 0.f;
    }
#pragma unroll
    for (int j = 0; j < kMaxMine; ++j) {
        if (j >= nmine) break;                            // warp-uniform
        const uint32_t kw[4] = {kraw[j].x, kraw[j].y, kraw[j].z, kraw[j].w};
        const uint32_t vw[4] = {vraw[j].x, vraw[j].y, vraw[j].z, vraw[j].w};
        float kf[8], vf[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 a = __half22float2(u32_as_h2(kw[i])), b = __half22float2(u32_as_h2(vw[i]));
            kf[2 * i] = a.x; kf[2 * i + 1] = a.y; vf[2 * i] = b.x; vf[2 * i + 1] = b.y;
        }
        const float cnt = (float)nval[j];
#pragma unroll
        for (int h = 0; h < 4; ++h) {
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(q[h][i], kf[i], s);
            if (hl >= LPV) s = 0.f;
#pragma unroll
            for (int o2 = 1; o2 < 16; o2 <<= 1) s += __shfl_xor_sync(0xffffffffu, s, o2);
            if (s > m[h]) {                               // exact running maximum (natural-log domain)
                const float corr = expf(m[h] - s);
                l[h] *= corr;
#pragma unroll
                for (int i = 0; i < 8; ++i) o[h][i] *= corr;
                m[h] = s;
            }
            const float w = expf(s - m[h]) * cnt;
            l[h] += w;
#pragma unroll
            for (int i = 0; i < 8; ++i) o[h][i] = fmaf(w, vf[i], o[h][i]);
            if (MASS && hl == 0 && h0 + h < p.rep) {     // the block's whole mass is reported as its first unit
                constexpr int UPB = kP / G;
                const int orig = (int)tab[warp + kConsumerWarps * j].w;
                float2* mp = p.mass_part + ((size_t)it.row * p.nb + orig) * UPB * p.rep + (h0 + h);
                mp[0] = make_float2(m[h], w);
                for (int u = 1; u < UPB; ++u) mp[(size_t)u * p.rep] = make_float2(-INFINITY, 0.f);
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 4; ++h) {
        if (h0 + h < p.rep && hl < LPV) {
            float* rec = rec0 + (size_t)(h0 + h) * (D + 2);
            if (hl == 0) { rec[0] = m[h]; rec[1] = l[h]; }
            float2* d2 = reinterpret_cast<float2*>(rec + 2 + 8 * hl);      // records are 8-byte aligned
            d2[0] = make_float2(o[h][0], o[h][1]); d2[1] = make_float2(o[h][2], o[h][3]);
            d2[2] = make_float2(o[h][4], o[h][5]); d2[3] = make_float2(o[h][6], o[h][7]);
        }
    }
}

template <int D, int G, bool DUP, bool MASS>
__device__ void consumer_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    Ctx<D, G> c;
    c.r = lane >> 2; c.t = lane & 3; c.lane = lane; c.f = 0.f;
    c.part = DUP && (c.r & 1);
    // Pair pr of the CTA belongs to stream pr & 1 and takes every third block of it; inside the
    // block the two warps share out the units of G tokens (a block with a single unit goes to the first).
    constexpr int UPB = kP / UU::U;                 // units per block
    const int pr = warp >> 1, half = warp & 1;
    const int stream = pr & 1;
    const int u0 = UPB >= 2 ? half * (UPB / 2) : 0;
    const int u1 = UPB >= 2 ? u0 + UPB / 2 : (half == 0 ? 1 : 0);
    int seq = pr >> 1;
    int code = 0;                                   // non-zero: a wait gave up
    for (int iseq = 0; code == 0; ++iseq) {
        const int is = iseq % kItemSlots, ib = iseq & 1;
        if (!mbar_wait(&sm.item_full[is], (uint32_t)(iseq / kItemSlots) & 1u)) { code = 2; break; }
        const ItemDesc it = sm.item[is];
        if (it.exit) return;
        if (!mbar_wait(&sm.qready[ib], (uint32_t)(iseq >> 1) & 1u)) { code = 3; break; }
        c.qprep = smem_u32(sm.qprep) + (uint32_t)(ib * C::QPREP_BYTES) + (uint32_t)lane * 16u;
        c.sq = smem_u32(sm.sq) + (uint32_t)(ib * C::SQ_BYTES);
        c.f = sm.sf[ib * 16 + head_of_row<DUP>(c.r)];
        const size_t rec_idx = (size_t)it.row * p.items_per_row + (size_t)(it.item / p.rows);
        float* rec0 = p.part + (rec_idx * kConsumerWarps + warp) * p.rep * (D + 2);
        if (it.level == 1) {
            centroid_item<D, G, MASS>(p, c, it, sm.item_tab + is * kMaxItemBlocks, warp, rec0);
        }
        else if (it.level == 16) code = ring_item<D, G, 16, DUP, MASS>(
                p, sm, c, it, stream, u0, u1, seq, rec0);
        else if (it.level == 8) code = ring_item<D, G, 8, DUP, MASS>(
                p, sm, c, it, stream, u0, u1, seq, rec0);
        else if (it.level == 4) code = ring_item<D, G, 4, DUP, MASS>(
                p, sm, c, it, stream, u0, u1, seq, rec0);
        else code = ring_item<D, G, 2, DUP, MASS>(
                p, sm, c, it, stream, u0, u1, seq, rec0);
        if (code) break;
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.item_empty[is]);
        if (*reinterpret_cast<volatile int*>(abort_flag)) return;
    }
    if (code && lane == 0) {
        atomicExch(p.status, code);
        atomicExch(abort_flag, 1);
    }
}

// MASS: the variant that also reports the blocks' softmax mass.  It is a separate instantiation because the few
// extra live values of the reporting measurably slow the plain kernel down (5 % on the 16k-token mix).
template <int D, int G, bool DUP, bool MASS>
__global__ void __launch_bounds__(kThreads, kCtasPerSM) decode_mma_kernel(const __grid_constant__ Params p,
                                                                         const __grid_constant__ TensorMaps tm) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    __shared__ int abort_flag;
    Smem<D, G> sm(smem_raw);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < kStreams * kNSlot; ++s) {
            mbar_init(&sm.full[s], 1 + 32);         // lane 0's arrival (+ bulk-copy bytes) and 32 scale-copy arrivals
            mbar_init(&sm.empty[s], 2);             // the two warps of a pair
        }
        for (int s = 0; s < kItemSlots; ++s) {
            mbar_init(&sm.item_full[s], 1);
            mbar_init(&sm.item_empty[s], kConsumerWarps + kStreams);
        }
        mbar_init(&sm.qready[0], 1);
        mbar_init(&sm.qready[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x < kConsumers) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kConsumerRegs));
    else asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kHelperRegs));
    if (threadIdx.x < kConsumers) consumer_loop<D, G, DUP, MASS>(p, sm, &abort_flag);
    // Warp w issues from scheduler w mod 4.  The consumers of stream 0 (pairs 0, 2, 4) sit on schedulers
    // 0 and 1, those of stream 1 on 2 and 3; each producer is put on a scheduler of its OWN stream, so
    // that it gets the issue slots exactly when its consumers are waiting for it.
    else if (threadIdx.x < kConsumers + 32) producer_loop<D, G>(p, tm, sm, 0, &abort_flag);        // warp 12: scheduler 0
    else if (threadIdx.x < kConsumers + 64) query_loop<D, G, DUP>(p, sm, &abort_flag);         // warp 13: scheduler 1
    else if (threadIdx.x < kConsumers + 96) producer_loop<D, G>(p, tm, sm, 1, &abort_flag);        // warp 14: scheduler 2
    else scheduler_loop<D, G>(p, sm, &abort_flag);                                             // warp 15: scheduler 3
}

}  // namespace mma
}  // namespace gkv
