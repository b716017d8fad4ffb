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
// Structure (one CTA = 4 consumer warps + 1 producer warp, two CTAs per SM, persistent):
//   * work items are (cache row, chunk of consecutive blocks), handed out by an atomic
//     counter; every item ends in one (m, l, o) record per query head of the row;
//   * the producer warp streams each block's bytes and its four scale planes into a byte
//     ring in shared memory with cp.async.bulk + mbarrier (non-multicast), several blocks
//     ahead of the consumers;
//   * consumer warp w takes the blocks whose position in the stream is w mod 4 and runs a
//     private online softmax over them; the four states are merged at the end of the item.
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
// bits; the lo terms are two tiny extra MMAs.  Accumulation is fp32 throughout.
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
#ifndef GKV_RING_KB
#define GKV_RING_KB 72    // byte ring per CTA
#endif
constexpr int kConsumerWarps = GKV_NW;
constexpr int kCtasPerSM = GKV_CTAS;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;
constexpr int kNSlot = kConsumerWarps <= 4 ? 16 : 32;   // descriptor slots (blocks in flight per CTA)
constexpr uint32_t kRingBytes = GKV_RING_KB * 1024;
constexpr unsigned long long kWaitLimitNs = 1000000000ull;  // every wait gives up after ~1 s, flags the error, returns

struct Desc {           // one block in the ring
    uint32_t off;       // byte offset of the block in the ring
    int32_t level;      // 0 = nothing to do (padding slot)
    int32_t nvalid;
    int32_t pad;
};

struct ItemDesc {       // one work item; published before any of its blocks so that the four
    int32_t item;       // consumer warps can meet at the item start without waiting for data
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
    float* part;        // (items, rep, D+2)
    int* counter;       // work-item counter (zeroed before launch)
    int* status;        // error word (zeroed before launch)
    int B, Hq, Hkv, nb, rep;
    int chunk;          // blocks per item
    int items_per_row, items;
    int per_row_meta;
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
    static constexpr int STAGE_FLOATS = kConsumerWarps * 8 * (D + 2);
    static constexpr size_t SMEM = kRingBytes + QPREP_BYTES + 8 * D * 4 + 64 + STAGE_FLOATS * 4 +
                                   kNSlot * sizeof(Desc) + 2 * kNSlot * 8 + 2 * sizeof(ItemDesc) + 5 * 8 + 64;
    static_assert(D % 32 == 0 && (G == 16 || G == 32 || G == 64) && D % G == 0, "unsupported shape");
};

template <int D, int G>
struct Smem {
    using C = Cfg<D, G>;
    uint8_t* ring;
    __half* qprep;
    float* sq;        // [8][D] raw query (fp32, softmax scale included)
    float* sf;        // [8] per-head factor 2^-eq * log2(e); [8..16) unused
    float* stage;
    Desc* desc;
    uint64_t* full;
    uint64_t* empty;
    ItemDesc* item;        // [2]
    uint64_t* item_full;   // [2]
    uint64_t* item_empty;  // [2]
    uint64_t* sync_bar;    // consumer rendezvous (4 arrivals: one per warp)
    __device__ explicit Smem(uint8_t* base) {
        ring = base;
        qprep = reinterpret_cast<__half*>(base + kRingBytes);
        sq = reinterpret_cast<float*>(base + kRingBytes + C::QPREP_BYTES);
        sf = sq + 8 * D;
        stage = sf + 16;
        desc = reinterpret_cast<Desc*>(stage + C::STAGE_FLOATS);
        full = reinterpret_cast<uint64_t*>(desc + kNSlot);
        empty = full + kNSlot;
        item_full = empty + kNSlot;
        item_empty = item_full + 2;
        sync_bar = item_empty + 2;
        item = reinterpret_cast<ItemDesc*>(sync_bar + 1);
    }
};

// ================================ producer ====================================================
// One lane does the streaming.  Per work item all 32 lanes fetch the metadata of the item's
// (<= 32) blocks in one coalesced pass and park it in a small shared table; lane 0 then walks
// the table: ring allocation, slot descriptor, expect-tx and the bulk copies of the block and
// of its four scale planes.  (An earlier version broadcast every block's metadata with warp
// shuffles; under the consumers' shared-memory traffic those cost ~1700 cycles per block and
// capped the whole kernel at 2.3 TB/s.)
template <int D, int G>
__device__ void producer_loop(const Params& p, Smem<D, G>& sm, int* abort_flag) {
    using C = Cfg<D, G>;
    const int lane = threadIdx.x & 31;
    __shared__ uint4 meta_tab[32];            // per block of the item: src offset (64 bit), level | nvalid << 8 | index << 16, bytes
    uint32_t head = 0, used = 0;
    int seq_alloc = 0, seq_free = 0;

    auto release_oldest = [&]() -> bool {     // lane 0 only
        const int s = seq_free % kNSlot;
        if (!mbar_wait(&sm.empty[s], (uint32_t)(seq_free / kNSlot) & 1u)) return false;
        used -= (uint32_t)sm.desc[s].pad;
        ++seq_free;
        return true;
    };

    int item = 0;
    if (lane == 0) item = atomicAdd(p.counter, 1);
    item = __shfl_sync(0xffffffffu, item, 0);
    bool ok = true;
    for (int iseq = 0; ok; ++iseq) {
        const bool done = item >= p.items;
        int next_item = 0;
        if (!done && lane == 0) next_item = atomicAdd(p.counter, 1);   // prefetch the next item id
        const int row = done ? 0 : item / p.items_per_row;
        const int b_lo = done ? 0 : (item % p.items_per_row) * p.chunk;
        const int nblk = done ? 0 : min(p.chunk, p.nb - b_lo);        // <= 32
        const int mrow = p.per_row_meta ? row : 0;
        // Blocks of an item are streamed sorted by rung (softmax does not care about the order):
        // the consumer warps of an SM then run the same unpack path at the same time, which
        // keeps the instruction cache warm.
        {
            int lv = 0, nv = 0;
            unsigned long long src = 0;
            if (lane < nblk) {
                const size_t mi = (size_t)mrow * p.nb + b_lo + lane;
                lv = p.level[mi];
                nv = min(p.valid[mi], kP);
                if (!level_ok(lv) || nv <= 0) lv = 0;
                src = (unsigned long long)row * (unsigned long long)p.stride_bh + (unsigned long long)p.offs[mi];
            }
            const int cls = lane >= nblk ? 6 : lv == 16 ? 0 : lv == 8 ? 1 : lv == 4 ? 2 : lv == 2 ? 3 : lv == 1 ? 4 : 5;
            int rank = 0;
#pragma unroll
            for (int c = 0; c < 6; ++c) {
                const unsigned m = __ballot_sync(0xffffffffu, cls == c);
                if (c < cls) rank += __popc(m);
                else if (c == cls) rank += __popc(m & ((1u << lane) - 1u));
            }
            if (lane < nblk) {
                const bool quant = lv == 8 || lv == 4 || lv == 2;
                const uint32_t bytes = (lv ? 2u * (uint32_t)half_bytes(lv, D) : 0u) + (quant ? 2u * (C::KSCALE + C::VSCALE) : 0u);
                meta_tab[rank] = make_uint4((uint32_t)src, (uint32_t)(src >> 32),
                                            (uint32_t)lv | ((uint32_t)max(nv, 0) << 8) | ((uint32_t)lane << 16), bytes);
            }
        }
        __syncwarp();
        if (lane == 0) {
            // the item descriptor goes out first, through its own double buffer
            const int ib = iseq & 1;
            if (iseq >= 2) ok = mbar_wait(&sm.item_empty[ib], (uint32_t)((iseq >> 1) - 1) & 1u);
            if (ok) {
                ItemDesc it;
                it.item = item; it.row = row; it.end_seq = seq_alloc + nblk; it.exit = done ? 1 : 0;
                sm.item[ib] = it;
                mbar_arrive(&sm.item_full[ib]);
            }
            const size_t sb0 = (size_t)row * p.nb + b_lo;
            uint4 e = meta_tab[0];
            for (int j = 0; j < nblk && ok; ++j) {
                const uint4 cur = e;
                if (j + 1 < nblk) e = meta_tab[j + 1];
                const int lvj = (int)(cur.z & 0xffu), nvj = (int)((cur.z >> 8) & 0xffu), orig = (int)(cur.z >> 16);
                const uint32_t bytes = cur.w;
                const uint32_t need = (bytes + 127u) & ~127u;
                const int slot = seq_alloc % kNSlot;
                while (ok && seq_alloc - seq_free >= kNSlot) ok = release_oldest();
                const uint32_t waste = (head + need > kRingBytes) ? kRingBytes - head : 0u;
                while (ok && used + waste + need > kRingBytes) ok = release_oldest();
                if (!ok) break;
                const uint32_t dst = waste ? 0u : head;
                used += waste + need;
                head = dst + need;
                if (head >= kRingBytes) head = 0;
                Desc d;
                d.off = dst; d.level = lvj; d.nvalid = nvj; d.pad = (int32_t)(waste + need);
                sm.desc[slot] = d;
                if (lvj) {
                    const bool quant = lvj == 8 || lvj == 4 || lvj == 2;
                    const uint32_t dbytes = 2u * (uint32_t)half_bytes(lvj, D);
                    const uint8_t* src = p.data + (((unsigned long long)cur.y << 32) | cur.x);
                    uint8_t* d0 = sm.ring + dst;
                    const size_t sb = sb0 + orig;
#ifdef GKV_DBG_NOLOAD
                    if (true) { mbar_arrive(&sm.full[slot]); } else
#endif
                    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                        mbar_arrive_tx(&sm.full[slot], bytes);
                        bulk_g2s(d0, src, dbytes, &sm.full[slot]);
                        if (quant) {
                            bulk_g2s(d0 + dbytes, p.klo + sb * (C::KSCALE / 2), C::KSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + C::KSCALE, p.kstep + sb * (C::KSCALE / 2), C::KSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + 2 * C::KSCALE, p.vlo + sb * (C::VSCALE / 2), C::VSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + 2 * C::KSCALE + C::VSCALE, p.vstep + sb * (C::VSCALE / 2), C::VSCALE, &sm.full[slot]);
                        }
                    } else {
                        // block start not 16-byte aligned (a cache row at an odd address): bulk copies
                        // cannot be used; this lane copies the block by hand, scale planes by bulk copy
                        for (uint32_t i = 0; i < dbytes; ++i) d0[i] = src[i];
                        __threadfence_block();
                        mbar_arrive_tx(&sm.full[slot], bytes - dbytes);    // the slot's single arrival
                        if (quant) {
                            bulk_g2s(d0 + dbytes, p.klo + sb * (C::KSCALE / 2), C::KSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + C::KSCALE, p.kstep + sb * (C::KSCALE / 2), C::KSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + 2 * C::KSCALE, p.vlo + sb * (C::VSCALE / 2), C::VSCALE, &sm.full[slot]);
                            bulk_g2s(d0 + dbytes + 2 * C::KSCALE + C::VSCALE, p.vstep + sb * (C::VSCALE / 2), C::VSCALE, &sm.full[slot]);
                        }
                    }
                } else {
                    mbar_arrive(&sm.full[slot]);
                }
                ++seq_alloc;
            }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        seq_alloc = __shfl_sync(0xffffffffu, seq_alloc, 0);
        if (!ok || done) break;
        item = __shfl_sync(0xffffffffu, next_item, 0);
    }
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

// Prepared-query fragment loader: plane pl, returns the 4 registers of chunk i (k-steps 2i, 2i+1).
template <int D, int G>
__device__ __forceinline__ uint4 load_qchunk(const Smem<D, G>& sm, int plane, int i, int lane) {
    using C = Cfg<D, G>;
    return *reinterpret_cast<const uint4*>(sm.qprep + (size_t)plane * C::QPLANE + ((size_t)i * 32 + lane) * 8);
}

// Rendezvous of the four consumer warps on an mbarrier (bounded, unlike bar.sync).
__device__ __forceinline__ bool consumer_sync(uint64_t* bar, uint32_t& phase) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
    const bool ok = mbar_wait(bar, phase);
    phase ^= 1u;
    return ok;
}

// Build the prepared query planes for the current row (all 128 consumer threads).
template <int D, int G>
__device__ bool prepare_query(const Params& p, Smem<D, G>& sm, int row, uint32_t& phase) {
    using C = Cfg<D, G>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = row / p.Hkv, hk = row % p.Hkv;
    const float* q = p.q + ((size_t)b * p.Hq + (size_t)hk * p.rep) * D;
    for (int i = tid; i < 8 * D; i += kConsumers) {
        const int h = i / D;
        sm.sq[i] = h < p.rep ? q[i] : 0.f;
    }
    if (!consumer_sync(sm.sync_bar, phase)) return false;
    // per-head power-of-two scale bringing max|q| into [8, 16): one head per warp at a time
    for (int h = warp; h < 8; h += kConsumerWarps) {
        float mx = 0.f;
        for (int d = lane; d < D; d += 32) mx = fmaxf(mx, fabsf(sm.sq[h * D + d]));
#pragma unroll
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        int eq = 0;
        if (mx > 0.f && mx < INFINITY) eq = 3 - ilogbf(mx);
        eq = max(-100, min(100, eq));
        if (lane == 0) {
            sm.sf[h] = ldexpf(1.4426950408889634f, -eq);
            sm.sf[8 + h] = ldexpf(1.0f, eq);
        }
    }
    if (!consumer_sync(sm.sync_bar, phase)) return false;
    // every thread fills entries (chunk i, lane l, half j) of each plane
    for (int idx = tid; idx < C::CH * 32 * 8; idx += kConsumers) {
        const int j = idx & 7, l = (idx >> 3) & 31, i = idx >> 8;
        const int r = l >> 2, t = l & 3;
        const int s = 2 * i + (j >> 2), e = j & 3;
        const float sc = sm.sf[8 + r];
#pragma unroll
        for (int a = 0; a < 3; ++a) {
            const int bits = a == 0 ? 8 : a == 1 ? 4 : 2;
            const float x = sm.sq[r * D + C::DT * t + arr_chan(bits, s, e)] * sc * arr_scale(bits, e);
            const __half h = __float2half_rn(x);
            sm.qprep[(2 * a) * C::QPLANE + idx] = h;
            sm.qprep[(2 * a + 1) * C::QPLANE + idx] = __float2half_rn(x - __half2float(h));
        }
        const float x = sm.sq[r * D + C::DT * t + arr_chan(16, s, e)] * sc;
        const __nv_bfloat16 hb = __float2bfloat16_rn(x);
        reinterpret_cast<__nv_bfloat16*>(sm.qprep)[6 * C::QPLANE + idx] = hb;
        reinterpret_cast<__nv_bfloat16*>(sm.qprep)[7 * C::QPLANE + idx] = __float2bfloat16_rn(x - __bfloat162float(hb));
    }
    return consumer_sync(sm.sync_bar, phase);
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

// ---- q . klo for every token group of a quantised block: one n-tile whose column n is group n ----
template <int D, int G>
__device__ __forceinline__ void key_bias(const Ctx<D, G>& c, uint32_t klo, float (&bias)[4]) {
    using C = Cfg<D, G>;
    const bool live = c.r < C::TG;
    const uint32_t lo = klo + (uint32_t)(((live ? c.r : 0) * D + C::DT * c.t) * 2);
    bias[0] = bias[1] = bias[2] = bias[3] = 0.f;
#pragma unroll
    for (int i = 0; i < C::CH; ++i) {
        const uint4 qh = qchunk(c, 0, i), ql = qchunk(c, 1, i);
        uint4 b = lds_v4(lo + 16 * i);
        if (!live) b = make_uint4(0, 0, 0, 0);
        mma_f16(bias, qh.x, ql.x, qh.y, ql.y, b.x, b.y);
        mma_f16(bias, qh.z, ql.z, qh.w, ql.w, b.z, b.w);
    }
}

// ---- K side of one unit of a quantised block: scores in the log2 domain ---------------------------
template <int D, int G, int BITS>
__device__ __forceinline__ void scores_unit(const Ctx<D, G>& c, uint32_t blk, int tg, const float (&bias)[4],
                                            float (&z)[Unit<D, G>::ZN]) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    constexpr int RB = D * BITS / 8;                     // bytes per token row
    constexpr int TB = RB / 4;                           // bytes per thread per row
    constexpr int plane = BITS == 8 ? 0 : BITS == 4 ? 2 : 4;
    const uint32_t nat = blk + (uint32_t)(2 * (kP * RB) + C::KSCALE + (tg * D + C::DT * c.t) * 2);
    const uint32_t row0 = blk + (uint32_t)((tg * UU::U + c.r) * RB + c.t * TB);

    float acc[UU::NU][4];
#pragma unroll
    for (int n = 0; n < UU::NU; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll 1
    for (int i = 0; i < C::CH; ++i) {                   // two k-steps at a time
        const uint4 qh = qchunk(c, plane, i), ql = qchunk(c, plane + 1, i);
        uint32_t sp[4];                                  // step pairs of k-steps 2i and 2i+1 in this arrangement
        if (BITS == 8) {
            const uint4 v = lds_v4(nat + 16 * i);
            sp[0] = v.x; sp[1] = v.y; sp[2] = v.z; sp[3] = v.w;
        } else if (BITS == 4) {                          // s = 2x+y with x = i: words 4i+y, 4i+y+2
            const uint4 v = lds_v4(nat + 16 * i);
            sp[0] = prmt(v.x, v.z, 0x5410); sp[1] = prmt(v.x, v.z, 0x7632);
            sp[2] = prmt(v.y, v.w, 0x5410); sp[3] = prmt(v.y, v.w, 0x7632);
        } else {                                         // s = 4x+y: x = i>>1, y = 2(i&1)+{0,1}: words 8x+y, 8x+y+4
            const uint32_t w0 = nat + (uint32_t)(32 * (i >> 1) + 8 * (i & 1));
            const uint2 va = lds_v2(w0), vb = lds_v2(w0 + 16);
            sp[0] = prmt(va.x, vb.x, 0x5410); sp[1] = prmt(va.x, vb.x, 0x7632);
            sp[2] = prmt(va.y, vb.y, 0x5410); sp[3] = prmt(va.y, vb.y, 0x7632);
        }
        uint32_t a[8];
        mul_split(qh.x, ql.x, sp[0], a[0], a[1]);
        mul_split(qh.y, ql.y, sp[1], a[2], a[3]);
        mul_split(qh.z, ql.z, sp[2], a[4], a[5]);
        mul_split(qh.w, ql.w, sp[3], a[6], a[7]);
        const uint32_t rowi = row0 + (uint32_t)(BITS == 8 ? 8 * i : BITS == 4 ? 4 * i : 4 * (i >> 1));
        const int sh2 = 8 * (i & 1);
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) {
            uint32_t b0, b1, b2, b3;                     // B registers of k-steps 2i (b0,b1) and 2i+1 (b2,b3)
            if (BITS == 8) {
                const uint2 w = lds_v2(rowi + n * 8 * RB);
                b0 = prmt(w.x, 0u, 0x4140); b1 = prmt(w.x, 0u, 0x4342);
                b2 = prmt(w.y, 0u, 0x4140); b3 = prmt(w.y, 0u, 0x4342);
            } else if (BITS == 4) {
                const uint32_t w = lds_u32(rowi + n * 8 * RB);
                const uint32_t u = w << 3, v = w >> 5;
                b0 = u & 0x00780078u; b1 = u & 0x07800780u;
                b2 = v & 0x00780078u; b3 = v & 0x07800780u;
            } else {
                // fields 4h..4h+3 (and +8) of the word, h = i & 1, brought to bits 8-9 / 6-7
                const uint32_t w = lds_u32(rowi + n * 8 * RB) >> sh2;
                const uint32_t u = w << 4;
                b0 = (w << 8) & 0x03000300u; b1 = u & 0x00C000C0u;
                b2 = u & 0x03000300u;        b3 = w & 0x00C000C0u;
            }
            mma_f16(acc[n], a[0], a[1], a[2], a[3], b0, b1);
            mma_f16(acc[n], a[4], a[5], a[6], a[7], b2, b3);
        }
    }
    // bias of this token group for head r lives in lane 4r + tg/2, column tg & 1
    const float bsel = (tg & 1) ? bias[1] + bias[3] : bias[0] + bias[2];
    const float bg = __shfl_sync(0xffffffffu, bsel, (c.lane & ~3) | (tg >> 1));
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
#pragma unroll
        for (int n = 0; n < UU::NU; ++n) {
            const uint4 w = lds_v4(row0 + 16 * i + n * 8 * D * 2);
            mma_bf16(acc[n], qh.x, ql.x, qh.y, ql.y, w.x, w.y);
            mma_bf16(acc[n], qh.z, ql.z, qh.w, ql.w, w.z, w.w);
        }
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
template <int D, int G>
__device__ __forceinline__ void softmax_unit(const Ctx<D, G>& c, WarpState<D, G>& st, float (&z)[Unit<D, G>::ZN], int nrel) {
    using UU = Unit<D, G>;
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < UU::ZN; ++i) {
        const int tok = (i >> 1) * 8 + 2 * c.t + (i & 1);
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

// Pairs (x[tok][cg], x[tok+1][cg]) of a (64, GV) fp16 plane at shared address `row` (token `tok`, even).
template <int GV>
__device__ __forceinline__ void scale_pairs(uint32_t row, uint32_t (&out)[GV]) {
    if (GV == 4) {
        const uint4 v = lds_v4(row);
        out[0] = prmt(v.x, v.z, 0x5410); out[1] = prmt(v.x, v.z, 0x7632);
        out[2 % GV] = prmt(v.y, v.w, 0x5410); out[3 % GV] = prmt(v.y, v.w, 0x7632);
    } else if (GV == 2) {
        const uint2 v = lds_v2(row);
        out[0] = prmt(v.x, v.y, 0x5410); out[1 % GV] = prmt(v.x, v.y, 0x7632);
    } else {
#pragma unroll
        for (int cg = 0; cg < GV; ++cg) out[cg] = lds_u16(row + 2 * cg) | (lds_u16(row + 2 * (GV + cg)) << 16);
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
    const int tok0 = unit * UU::U + 2 * c.t;         // first token of this thread's pair in k-step 0
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
        scale_pairs<C::GV>(srow + C::VSCALE, sa);                     // vstep, tokens (ta, ta+1)
        scale_pairs<C::GV>(srow + C::VSCALE + 8 * C::GV * 2, sb);     // vstep, tokens (tb, tb+1)
        scale_pairs<C::GV>(srow, la);                                 // vlo
        scale_pairs<C::GV>(srow + 8 * C::GV * 2, lb);
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
                const uint32_t src = vrow + (uint32_t)(((k & 2) ? 8 : 0) * RB + (k & 1) * RB + (G * cg * BITS) / 8);
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

// One quantised block: bias once, then its units.
template <int D, int G, int BITS>
__device__ __forceinline__ void quant_block(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int nvalid) {
    using C = Cfg<D, G>;
    using UU = Unit<D, G>;
    float bias[4];
    key_bias(c, blk + 2 * (kP * D * BITS / 8), bias);
#pragma unroll 1
    for (int unit = 0; unit < kP / UU::U; ++unit) {
        const int nrel = nvalid - unit * UU::U;
        if (nrel <= 0) break;
        float z[UU::ZN];
        scores_unit<D, G, BITS>(c, blk, unit, bias, z);
        softmax_unit(c, st, z, nrel);
        values_unit<D, G, BITS>(c, st, blk, unit, z);
    }
}

template <int D, int G>
__device__ __forceinline__ void bf16_block(const Ctx<D, G>& c, WarpState<D, G>& st, uint32_t blk, int nvalid) {
    using UU = Unit<D, G>;
#pragma unroll 1
    for (int unit = 0; unit < kP / UU::U; ++unit) {
        const int nrel = nvalid - unit * UU::U;
        if (nrel <= 0) break;
        float z[UU::ZN];
        scores_unit_bf16(c, blk, unit, z);
        softmax_unit(c, st, z, nrel);
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
__device__ void consumer_loop(const Params& p, Smem<D, G>& sm, int* abort_flag, int* next_seq) {
    using C = Cfg<D, G>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int r = lane >> 2, t = lane & 3;
    WarpState<D, G> st;
    Ctx<D, G> c;
    c.qprep = smem_u32(sm.qprep) + (uint32_t)lane * 16u;
    c.sq = smem_u32(sm.sq);
    c.r = r; c.t = t; c.lane = lane; c.f = 0.f;
    const uint32_t ring = smem_u32(sm.ring);
    uint32_t sync_phase = 0;
    // Blocks are taken from the stream dynamically: whichever warp is free grabs the next
    // position (block sizes span 64x, a fixed round-robin left warps idle at every item end).
    auto grab = [&]() -> int {
        int v = 0;
        if (lane == 0) v = atomicAdd(next_seq, 1);
        return __shfl_sync(0xffffffffu, v, 0);
    };
    int seq = grab();
    int code = 0;                                   // non-zero: a wait gave up
    for (int iseq = 0; code == 0; ++iseq) {
        const int ib = iseq & 1;
        if (!mbar_wait(&sm.item_full[ib], (uint32_t)(iseq >> 1) & 1u)) { code = 2; break; }
        const ItemDesc it = sm.item[ib];
        if (it.exit) return;
#ifndef GKV_DBG_NOITEM
        if (!prepare_query(p, sm, it.row, sync_phase)) { code = 3; break; }
#endif
#pragma unroll
        for (int n = 0; n < C::NTILE; ++n) st.o[n][0] = st.o[n][1] = st.o[n][2] = st.o[n][3] = 0.f;
        st.ob[0] = st.ob[1] = st.ob[2] = st.ob[3] = 0.f;
        st.m = -INFINITY;
        st.l = 0.f;
        c.f = sm.sf[r];

        for (; seq < it.end_seq; seq = grab()) {
            const int slot = seq % kNSlot;
            if (!mbar_wait(&sm.full[slot], (uint32_t)(seq / kNSlot) & 1u)) { code = 4; break; }
            const Desc d = sm.desc[slot];
#ifdef GKV_DBG_NOCOMPUTE
            if (false) {
#else
            if (d.level) {
#endif
                const uint32_t blk = ring + d.off;
                if (d.nvalid < kP && d.level != 1) clear_invalid_tail<D, G>(sm.ring + d.off, d.level, d.nvalid, lane);
                if (d.level == 1) centroid_block(c, st, blk, d.nvalid);
                else if (d.level == 16) bf16_block(c, st, blk, d.nvalid);
                else if (d.level == 8) quant_block<D, G, 8>(c, st, blk, d.nvalid);
                else if (d.level == 4) quant_block<D, G, 4>(c, st, blk, d.nvalid);
                else quant_block<D, G, 2>(c, st, blk, d.nvalid);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[slot]);
        }
        if (code) break;

#ifdef GKV_DBG_NOITEM
        if (tid == 0) mbar_arrive(&sm.item_empty[ib]);
        continue;
#endif
        // ---- merge the four warp states of this item and write its record ----------------------
        float l = st.l;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        float* mine = sm.stage + (size_t)warp * 8 * (D + 2) + (size_t)r * (D + 2);
        if (t == 0) { mine[0] = st.m; mine[1] = l; }
        // p . vlo of channel group cg sits in lane 4r + cg/2, column cg & 1, scaled 2^8
        const float ob_even = st.ob[0] + st.ob[2], ob_odd = st.ob[1] + st.ob[3];
#pragma unroll
        for (int cg = 0; cg < C::GV; ++cg) {
            const float src = (cg & 1) ? ob_odd : ob_even;
            const float bias = __shfl_sync(0xffffffffu, src, (lane & ~3) | (cg >> 1)) * 0.00390625f;
#pragma unroll
            for (int i = 0; i < C::NT; ++i) {
                const int n = cg * C::NT + i;
                mine[2 + G * cg + C::NT * (2 * t) + i] = fmaf(st.o[n][0] + st.o[n][2], 65536.f, bias);
                mine[2 + G * cg + C::NT * (2 * t + 1) + i] = fmaf(st.o[n][1] + st.o[n][3], 65536.f, bias);
            }
        }
        if (!consumer_sync(sm.sync_bar, sync_phase)) { code = 5; break; }
        float* rec = p.part + (size_t)it.item * p.rep * (D + 2);
        for (int h = warp; h < p.rep; h += kConsumerWarps) {
            float mw[kConsumerWarps], mmax = -INFINITY;
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                mw[w] = sm.stage[(size_t)w * 8 * (D + 2) + (size_t)h * (D + 2)];
                mmax = fmaxf(mmax, mw[w]);
            }
            float lsum = 0.f, wgt[kConsumerWarps];
#pragma unroll
            for (int w = 0; w < kConsumerWarps; ++w) {
                wgt[w] = (mw[w] == -INFINITY) ? 0.f : ex2(mw[w] - mmax);
                lsum += wgt[w] * sm.stage[(size_t)w * 8 * (D + 2) + (size_t)h * (D + 2) + 1];
            }
            for (int dd = lane; dd < D; dd += 32) {
                float a = 0.f;
#pragma unroll
                for (int w = 0; w < kConsumerWarps; ++w)
                    a = fmaf(wgt[w], sm.stage[(size_t)w * 8 * (D + 2) + (size_t)h * (D + 2) + 2 + dd], a);
                rec[(size_t)h * (D + 2) + 2 + dd] = a;
            }
            if (lane == 0) {
                // records are kept in the natural-log domain like the generic kernel's
                rec[(size_t)h * (D + 2) + 0] = mmax * 0.6931471805599453f;
                rec[(size_t)h * (D + 2) + 1] = lsum;
            }
        }
        if (!consumer_sync(sm.sync_bar, sync_phase)) { code = 6; break; }
        if (tid == 0) mbar_arrive(&sm.item_empty[ib]);
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
    __shared__ int abort_flag, next_seq;
    Smem<D, G> sm(smem_raw);
    if (threadIdx.x == 0) {
        abort_flag = 0;
        next_seq = 0;
        for (int s = 0; s < kNSlot; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.item_full[s], 1);
            mbar_init(&sm.item_empty[s], 1);
        }
        mbar_init(sm.sync_bar, kConsumerWarps);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x >= kConsumers) producer_loop<D, G>(p, sm, &abort_flag);
    else consumer_loop<D, G>(p, sm, &abort_flag, &next_seq);
}

}  // namespace mma
}  // namespace gkv
