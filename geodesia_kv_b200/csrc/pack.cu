// Pack, demote and unpack kernels for the bit-ladder block format.
//
// One CTA owns one block of one cache row.  The block's K and V are first brought into
// shared memory as fp32 tiles (rows padded by one float: the V groups are read along a row by
// threads that sit a whole group apart, which without the pad would all hit one bank) (from dense inputs when packing, from the packed bytes at the
// current rung when demoting — so no dense copy of the cache ever exists in global memory),
// then re-expressed at the target rung with exactly the arithmetic of the reference's
// quantize_codes (tests/test_cuda_kernel.py:18-33): fp32 min/max per group, step =
// max(hi-lo, 1e-8)/(2^b-1) with IEEE division, lo and step rounded to fp16 BEFORE the codes
// are taken, code = clamp(rint((x-lo16)/step16), 0, 2^b-1), codes packed little-endian in the
// byte (geodesia_kv/packed.py:23-40).  This file is compiled without fast-math.
//
// Head dims 64 and 128 (with a group that is a multiple of 8) take the register-resident path of
// requantise.cuh instead: no fp32 tile in shared memory, every load of the block in flight at once.
// The tile kernels below remain for the other shapes.
//
// Two addressings share the block code: cache ROWS (a byte string per row, dense scale tensors
// (rows, nb, ...) beside it — the reference's layout) and a paged POOL (every block an offset into
// one byte pool, the four scale planes of a quantised block stored right behind its bytes as
// [klo][kstep][vlo][vstep], so a block moves, shrinks and is freed as one piece).
#include "gkv_common.cuh"
#include "requantise.cuh"

namespace gkv {

constexpr int kPackThreads = 256;

struct TileJob {
    uint8_t* dst;          // block start in the destination row
    __half* klo; __half* kstep; __half* vlo; __half* vstep;   // this block's scale planes
    int level, D, group, G, gv;
    int ld;                // row stride of the fp32 tiles in floats
};

__host__ __device__ __forceinline__ int tile_ld(int D) { return D + 1; }

// code = clamp(rint((x - lo) / step), 0, qmax) with the quotient rounded as IEEE division rounds it.
// A correctly rounded division is ~10 instructions; the product with a reciprocal is within a
// few ulp of it (absolute error < 1e-4 for quotients up to 255), so it rounds to the same integer
// unless it lands within 1e-3 of a tie, and only then is the exact division needed.
__device__ __forceinline__ uint8_t exact_code(float x, float lf, float sf, float rs, float qmax) {
    const float a = __fsub_rn(x, lf);
    float q = __fmul_rn(a, rs);
    const float fr = q - floorf(q);
    if (!(fabsf(fr - 0.5f) > 1e-3f) || !(fabsf(q) < 1e6f)) q = __fdiv_rn(a, sf);    // near a tie, huge, or NaN
    float c = rintf(q);
    c = (c != c) ? 0.f : fminf(fmaxf(c, 0.f), qmax);
    return (uint8_t)c;
}

// Tiles: sk, sv hold [64][ld] fp32.  scode is a dense [64][D] byte scratch.
__device__ void quantize_tile_and_store(const TileJob& j, const float* __restrict__ sk,
                                        const float* __restrict__ sv, uint8_t* __restrict__ scode) {
    const int tid = threadIdx.x, D = j.D, lv = j.level, ld = j.ld;
    const int hb = half_bytes(lv, D);
    const bool scales_needed = (lv == 8 || lv == 4 || lv == 2);
    if (!scales_needed) {
        // the reference keeps zero scale planes for rungs 16 and 1 (pack_layout.py:25-28)
        for (int i = tid; i < j.G * D; i += kPackThreads) { j.klo[i] = __ushort_as_half(0); j.kstep[i] = __ushort_as_half(0); }
        for (int i = tid; i < kP * j.gv; i += kPackThreads) { j.vlo[i] = __ushort_as_half(0); j.vstep[i] = __ushort_as_half(0); }
    }
    if (lv == 16) {
        __nv_bfloat16* ko = reinterpret_cast<__nv_bfloat16*>(j.dst);
        __nv_bfloat16* vo = reinterpret_cast<__nv_bfloat16*>(j.dst + hb);
        // two channels per thread and store
        __nv_bfloat162* ko2 = reinterpret_cast<__nv_bfloat162*>(ko);
        __nv_bfloat162* vo2 = reinterpret_cast<__nv_bfloat162*>(vo);
        for (int i = tid; i < kP * D / 2; i += kPackThreads) {
            const int t = (2 * i) / D, d = 2 * i - t * D;
            ko2[i] = __floats2bfloat162_rn(sk[t * ld + d], sk[t * ld + d + 1]);
            vo2[i] = __floats2bfloat162_rn(sv[t * ld + d], sv[t * ld + d + 1]);
        }
        return;
    }
    if (lv == 1) {
        // mean over the 64 tokens: fp32, tokens added in order, one division
        __half* ko = reinterpret_cast<__half*>(j.dst);
        __half* vo = reinterpret_cast<__half*>(j.dst + hb);
        for (int d = tid; d < 2 * D; d += kPackThreads) {
            const float* src = d < D ? sk + d : sv + (d - D);
            float s = 0.f;
            for (int t = 0; t < kP; ++t) s = __fadd_rn(s, src[t * ld]);
            const __half h = __float2half_rn(__fdiv_rn(s, (float)kP));
            if (d < D) ko[d] = h; else vo[d - D] = h;
        }
        return;
    }
    const float qmax = (float)((1 << lv) - 1);
    const int per = 8 / lv;
    for (int which = 0; which < 2; ++which) {
        const float* src = which ? sv : sk;
        if (which == 0) {
            // K: per channel over groups of g consecutive tokens; scales (G, D)
            const int g = min(j.group, kP);
            for (int u = tid; u < j.G * D; u += kPackThreads) {
                const int tg = u / D, d = u - tg * D;
                float lo = INFINITY, hi = -INFINITY;
                for (int i = 0; i < g; ++i) {
                    const float x = src[(tg * g + i) * ld + d];
                    lo = fminf(lo, x); hi = fmaxf(hi, x);
                }
                const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
                const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
                j.klo[u] = l16; j.kstep[u] = s16;
                const float lf = __half2float(l16), sf = __half2float(s16), rs = __frcp_rn(sf);
                for (int i = 0; i < g; ++i) {
                    const int t = tg * g + i;
                    scode[t * D + d] = exact_code(src[t * ld + d], lf, sf, rs, qmax);
                }
            }
        } else {
            // V: per token over groups of g consecutive channels; scales (P, gv)
            const int g = min(j.group, D);
            for (int u = tid; u < kP * j.gv; u += kPackThreads) {
                const int t = u / j.gv, cg = u - t * j.gv;
                float lo = INFINITY, hi = -INFINITY;
                for (int i = 0; i < g; ++i) {
                    const float x = src[t * ld + cg * g + i];
                    lo = fminf(lo, x); hi = fmaxf(hi, x);
                }
                const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
                const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
                j.vlo[u] = l16; j.vstep[u] = s16;
                const float lf = __half2float(l16), sf = __half2float(s16), rs = __frcp_rn(sf);
                for (int i = 0; i < g; ++i) {
                    const int d = cg * g + i;
                    scode[t * D + d] = exact_code(src[t * ld + d], lf, sf, rs, qmax);
                }
            }
        }
        __syncthreads();
        uint8_t* out = j.dst + which * hb;
        if ((reinterpret_cast<uintptr_t>(out) & 3) == 0) {
            // four output bytes per thread and store (hb is a multiple of 4 for every D % 8 == 0)
            uint32_t* out4 = reinterpret_cast<uint32_t*>(out);
            for (int w = tid; w < hb / 4; w += kPackThreads) {
                uint32_t word = 0;
                for (int b = 0; b < 4; ++b) {
                    uint32_t byte = 0;
                    for (int i = 0; i < per; ++i) byte |= (uint32_t)scode[(4 * w + b) * per + i] << (i * lv);
                    word |= byte << (8 * b);
                }
                out4[w] = word;
            }
        } else {
            for (int o = tid; o < hb; o += kPackThreads) {
                uint32_t byte = 0;
                for (int i = 0; i < per; ++i) byte |= (uint32_t)scode[o * per + i] << (i * lv);
                out[o] = (uint8_t)byte;
            }
        }
        __syncthreads();
    }
}

// Exact dequantisation of one block into the fp32 tiles (mixed_attn.cu:93-159).
__device__ void dequant_block_to_tiles(const uint8_t* __restrict__ blk, int lv, int D, int group, int gv,
                                       const __half* klo, const __half* kstep, const __half* vlo,
                                       const __half* vstep, float* sk, float* sv, int ld) {
    const uint8_t* vb = blk + half_bytes(lv, D);
    for (int e = threadIdx.x; e < kP * D; e += blockDim.x) {
        const int t = e / D, d = e - t * D;
        float kx, vx;
        if (lv == 1) {
            kx = half_bits_to_float(reinterpret_cast<const uint16_t*>(blk)[d]);
            vx = half_bits_to_float(reinterpret_cast<const uint16_t*>(vb)[d]);
        } else if (lv == 16) {
            kx = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(blk)[e]);
            vx = bf16_bits_to_float(reinterpret_cast<const uint16_t*>(vb)[e]);
        } else {
            const int ks = (t / group) * D + d, vs = t * gv + d / group;
            kx = __fmaf_rn((float)unpack_code(blk, e, lv), __half2float(kstep[ks]), __half2float(klo[ks]));
            vx = __fmaf_rn((float)unpack_code(vb, e, lv), __half2float(vstep[vs]), __half2float(vlo[vs]));
        }
        sk[t * ld + d] = kx;
        sv[t * ld + d] = vx;
    }
}

struct PackParams {
    const void* k; const void* v; int src_dtype;
    uint8_t* data; const int64_t* offs;
    __half* klo; __half* kstep; __half* vlo; __half* vstep;
    const int32_t* level; const int32_t* valid;
    int nb, b_lo, D, group, G, gv, per_row_meta;
    int64_t stride_bh;
    int nbx;                // blocks per row handled by this launch (b_hi - b_lo)
};

__device__ __forceinline__ float load_src(const void* p, int dtype, size_t i) {
    if (dtype == 0) return static_cast<const float*>(p)[i];
    if (dtype == 1) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
    return __half2float(static_cast<const __half*>(p)[i]);
}

__global__ void __launch_bounds__(kPackThreads) pack_blocks_kernel(PackParams p) {
    extern __shared__ float smem[];
    const int D = p.D;
    const int ld = tile_ld(D);
    float* sk = smem;
    float* sv = sk + kP * ld;
    uint8_t* scode = reinterpret_cast<uint8_t*>(sv + kP * ld);
    const int blk = p.b_lo + blockIdx.x, row = blockIdx.y;
    const int mrow = p.per_row_meta ? row : 0;
    const int lv = p.level[(size_t)mrow * p.nb + blk];
    if (!level_ok(lv)) return;
    int nvalid = p.valid ? p.valid[(size_t)mrow * p.nb + blk] : kP;
    nvalid = max(1, min(nvalid, kP));
    const size_t src0 = ((size_t)row * p.nb + blk) * kP * D;
    const bool vec16 = p.src_dtype != 0 && ((reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0;
    if (vec16) {
        // eight 16-bit elements per load (D % 8 == 0, so a load never straddles a row)
        const uint4* k8 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.k) + src0);
        const uint4* v8 = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(p.v) + src0);
        for (int e8 = threadIdx.x; e8 < kP * D / 8; e8 += kPackThreads) {
            const int t = (8 * e8) / D, d = 8 * e8 - t * D;
            const int ts = min(t, nvalid - 1);           // pad by repeating the last real row
            const uint4 a = k8[(ts * D + d) / 8], b = v8[(ts * D + d) / 8];
            const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint16_t a0 = (uint16_t)(aw[i] & 0xffffu), a1 = (uint16_t)(aw[i] >> 16);
                const uint16_t b0 = (uint16_t)(bw[i] & 0xffffu), b1 = (uint16_t)(bw[i] >> 16);
                if (p.src_dtype == 1) {
                    sk[t * ld + d + 2 * i] = bf16_bits_to_float(a0); sk[t * ld + d + 2 * i + 1] = bf16_bits_to_float(a1);
                    sv[t * ld + d + 2 * i] = bf16_bits_to_float(b0); sv[t * ld + d + 2 * i + 1] = bf16_bits_to_float(b1);
                } else {
                    sk[t * ld + d + 2 * i] = half_bits_to_float(a0); sk[t * ld + d + 2 * i + 1] = half_bits_to_float(a1);
                    sv[t * ld + d + 2 * i] = half_bits_to_float(b0); sv[t * ld + d + 2 * i + 1] = half_bits_to_float(b1);
                }
            }
        }
    } else {
        for (int e = threadIdx.x; e < kP * D; e += kPackThreads) {
            const int t = e / D, d = e - t * D;
            const int ts = min(t, nvalid - 1);           // pad by repeating the last real row
            sk[t * ld + d] = load_src(p.k, p.src_dtype, src0 + (size_t)ts * D + d);
            sv[t * ld + d] = load_src(p.v, p.src_dtype, src0 + (size_t)ts * D + d);
        }
    }
    __syncthreads();
    TileJob j;
    j.dst = p.data + (size_t)row * p.stride_bh + p.offs[(size_t)mrow * p.nb + blk];
    const size_t sb = (size_t)row * p.nb + blk;
    j.klo = p.klo + sb * p.G * D; j.kstep = p.kstep + sb * p.G * D;
    j.vlo = p.vlo + sb * kP * p.gv; j.vstep = p.vstep + sb * kP * p.gv;
    j.level = lv; j.D = D; j.group = p.group; j.G = p.G; j.gv = p.gv; j.ld = ld;
    quantize_tile_and_store(j, sk, sv, scode);
}

struct DemoteParams {
    const uint8_t* data_old; const int64_t* offs_old; const int32_t* level_old;
    uint8_t* data_new; const int64_t* offs_new; const int32_t* level_new;
    __half* klo; __half* kstep; __half* vlo; __half* vstep;
    int nb, D, group, G, gv, per_row_meta;
    int64_t stride_old, stride_new;
};

__global__ void __launch_bounds__(kPackThreads) demote_blocks_kernel(DemoteParams p) {
    extern __shared__ float smem[];
    const int D = p.D;
    const int ld = tile_ld(D);
    float* sk = smem;
    float* sv = sk + kP * ld;
    uint8_t* scode = reinterpret_cast<uint8_t*>(sv + kP * ld);
    const int blk = blockIdx.x, row = blockIdx.y;
    const int mrow = p.per_row_meta ? row : 0;
    const size_t mi = (size_t)mrow * p.nb + blk;
    const int lo = p.level_old[mi], ln = p.level_new[mi];
    if (lo == ln || !level_ok(lo) || !level_ok(ln) || ln > lo) return;   // never promote
    const size_t sb = (size_t)row * p.nb + blk;
    TileJob j;
    j.klo = p.klo + sb * p.G * D; j.kstep = p.kstep + sb * p.G * D;
    j.vlo = p.vlo + sb * kP * p.gv; j.vstep = p.vstep + sb * kP * p.gv;
    dequant_block_to_tiles(p.data_old + (size_t)row * p.stride_old + p.offs_old[mi], lo, D, p.group, p.gv,
                           j.klo, j.kstep, j.vlo, j.vstep, sk, sv, ld);
    __syncthreads();
    j.dst = p.data_new + (size_t)row * p.stride_new + p.offs_new[mi];
    j.level = ln; j.D = D; j.group = p.group; j.G = p.G; j.gv = p.gv; j.ld = ld;
    quantize_tile_and_store(j, sk, sv, scode);
}

struct UnpackParams {
    const uint8_t* data; const int64_t* offs;
    const __half* klo; const __half* kstep; const __half* vlo; const __half* vstep;
    const int32_t* level; float* k_out; float* v_out;
    int nb, D, group, G, gv, per_row_meta;
    int64_t stride_bh;
};

__global__ void __launch_bounds__(kPackThreads) unpack_blocks_kernel(UnpackParams p) {
    const int blk = blockIdx.x, row = blockIdx.y, D = p.D;
    const int mrow = p.per_row_meta ? row : 0;
    const size_t mi = (size_t)mrow * p.nb + blk;
    const int lv = p.level[mi];
    if (!level_ok(lv)) return;
    const size_t sb = (size_t)row * p.nb + blk;
    dequant_block_to_tiles(p.data + (size_t)row * p.stride_bh + p.offs[mi], lv, D, p.group, p.gv,
                           p.klo + sb * p.G * D, p.kstep + sb * p.G * D, p.vlo + sb * kP * p.gv,
                           p.vstep + sb * kP * p.gv, p.k_out + sb * kP * D, p.v_out + sb * kP * D, D);
}


// Scale planes of a block of the paged pool: right behind the block's bytes.
__device__ __forceinline__ void scales_behind(const uint8_t* blk, int lv, int D, int G, int gv, const __half*& klo,
                                              const __half*& kstep, const __half*& vlo, const __half*& vstep) {
    const __half* base = reinterpret_cast<const __half*>(blk + 2 * half_bytes(lv, D));
    klo = base; kstep = klo + G * D; vlo = kstep + G * D; vstep = vlo + kP * gv;
}

struct PagedPackParams {
    const void* k; const void* v; int src_dtype;
    const int64_t* src_off; int64_t token_stride; const int32_t* nvalid;
    uint8_t* pool; const int64_t* dst_off; const int32_t* level;
    float* ek; float* ev;
    int group, G, gv;
};

struct PagedDemoteParams {
    const uint8_t* pool_old; uint8_t* pool_new;
    const int64_t* off_old; const int32_t* level_old;
    const int64_t* off_new; const int32_t* level_new;
    float* ek; float* ev;
    int group, G, gv;
};

struct PagedUnpackParams {
    const uint8_t* pool; const int64_t* offs; const int32_t* level; float* k_out; float* v_out;
    int D, group, G, gv;
};

__global__ void __launch_bounds__(kPackThreads) paged_unpack_kernel(PagedUnpackParams p) {
    const int i = blockIdx.x, D = p.D;
    const int lv = p.level[i];
    const int64_t off = p.offs[i];
    if (!level_ok(lv) || off < 0) return;
    const __half *klo, *kstep, *vlo, *vstep;
    scales_behind(p.pool + off, lv, D, p.G, p.gv, klo, kstep, vlo, vstep);
    dequant_block_to_tiles(p.pool + off, lv, D, p.group, p.gv, klo, kstep, vlo, vstep,
                           p.k_out + (size_t)i * kP * D, p.v_out + (size_t)i * kP * D, D);
}


// One new token per cache row, written into the row's open rung-16 block (bf16 rows, so an append is a
// plain store of two rows of D values) — the block table, the valid count and the row length are
// advanced on the device, so a decode step needs no host work unless a row starts a new block.
struct AppendParams {
    const void* k; const void* v; int src_dtype;
    uint8_t* pool; const int64_t* offs; int32_t* valid; int32_t* lens; int32_t* status;
    int cap, D;
};

__global__ void paged_append_kernel(AppendParams p) {
    const int row = blockIdx.x, D = p.D;
    const int len = p.lens[row];
    const int blk = len / kP, t = len - blk * kP;
    const int64_t off = blk < p.cap ? p.offs[(size_t)row * p.cap + blk] : -1;
    __syncthreads();                                   // every thread has read the length
    if (off < 0) {                                     // no slot was provided for the row's next block
        if (threadIdx.x == 0) atomicExch(p.status, 1);
        return;
    }
    __nv_bfloat16* kd = reinterpret_cast<__nv_bfloat16*>(p.pool + off) + (size_t)t * D;
    __nv_bfloat16* vd = kd + (size_t)kP * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        kd[d] = __float2bfloat16_rn(load_src(p.k, p.src_dtype, (size_t)row * D + d));
        vd[d] = __float2bfloat16_rn(load_src(p.v, p.src_dtype, (size_t)row * D + d));
    }
    if (threadIdx.x == 0) {
        p.valid[(size_t)row * p.cap + blk] = t + 1;
        p.lens[row] = len + 1;
    }
}


// ---- persistent, bulk-copy-fed kernels ---------------------------------------------------------------
// The kernels above start a CTA per block: the CTA reads the block's table entries, then its bytes, then
// computes, then stores — a chain of dependent memory round trips that two resident CTAs per SM cannot
// hide.  Here CTAs are persistent (two per SM) and hold a ninth warp, the producer: it looks up block
// i + grid (table entries: two dependent global loads) and starts ONE bulk copy per contiguous piece of
// its source (K rows, V rows; or the packed block and its scale planes) into a two-stage ring in shared
// memory while the 256 working threads are on block i out of the other stage, so every global-memory
// latency is overlapped with arithmetic.  Sources that a bulk copy cannot take
// (fp32 rows, a token stride other than D, an address that is not 16-byte aligned) are processed
// straight from global memory by the same CTA.
namespace st {

constexpr int kStages = 2;
constexpr int kTileBytes = 2 * kP * 128 * 2;          // the largest block: rung 16 at D = 128
constexpr int kScaleBytes = 4 * 4 * 128 * 2;          // four planes of at most (4, 128) fp16
constexpr int kStageBytes = kTileBytes + kScaleBytes;
constexpr unsigned long long kWaitNs = 2000000000ull; // a copy that has not landed after 2 s never will

struct Desc {
    int skip, staged, src_kind, nvalid, old_level, level, zero_scales, pad;
    const void* ksrc; const void* vsrc; long long src_stride;
    const uint8_t* old_blk; const __half* oklo; const __half* okstep; const __half* ovlo; const __half* ovstep;
    uint8_t* dst; __half* klo; __half* kstep; __half* vlo; __half* vstep; float* ek; float* ev;
};

struct __align__(128) Smem {
    rq::Shared work;
    Desc desc[kStages];
    unsigned long long full[kStages];
    unsigned long long empty[kStages];
    __align__(128) uint8_t stage[kStages][kStageBytes];
};

__device__ int g_status;        // set when a wait on a bulk copy ran out

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(unsigned long long* b, int n) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n));
}
__device__ __forceinline__ void bar_expect(unsigned long long* b, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bar_arrive(unsigned long long* b) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(b)) : "memory");
}
__device__ __forceinline__ bool bar_wait(unsigned long long* b, uint32_t parity) {
    unsigned long long t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
        uint32_t ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
                     : "=r"(ok) : "r"(s32(b)), "r"(parity), "r"(2000u) : "memory");
        if (ok) return true;
        if (spin > 1) __nanosleep(spin < 16 ? 100 : 400);      // a polling lane must not eat the workers' issue slots
        if ((spin & 63u) == 63u) {
            unsigned long long now;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
            if (t0 == 0) t0 = now;
            else if (now - t0 > kWaitNs) return false;
        }
    }
}
__device__ __forceinline__ void bulk(void* dst, const void* src, uint32_t bytes, unsigned long long* b) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(b)) : "memory");
}
__device__ __forceinline__ bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- what block i of each kind of launch is ----------------------------------------------------------
__device__ __forceinline__ void clear(Desc& d) {
    d.skip = 0; d.staged = 0; d.src_kind = 0; d.nvalid = kP; d.old_level = 0; d.level = 0; d.zero_scales = 0; d.pad = 0;
    d.ksrc = d.vsrc = nullptr; d.src_stride = 0; d.old_blk = nullptr; d.oklo = d.okstep = d.ovlo = d.ovstep = nullptr;
    d.dst = nullptr; d.klo = d.kstep = d.vlo = d.vstep = nullptr; d.ek = d.ev = nullptr;
}

template <int D>
__device__ void describe(const PackParams& p, int i, Desc& d) {
    clear(d);
    const int row = i / p.nbx, blk = p.b_lo + (i - row * p.nbx);
    const int mrow = p.per_row_meta ? row : 0;
    const size_t mi = (size_t)mrow * p.nb + blk;
    const int lv = p.level[mi];
    if (!level_ok(lv)) { d.skip = 1; return; }
    const size_t src0 = ((size_t)row * p.nb + blk) * kP * D, esz = p.src_dtype == 0 ? 4 : 2;
    d.src_kind = p.src_dtype; d.src_stride = D;
    d.nvalid = max(1, min(p.valid ? p.valid[mi] : kP, kP));
    d.ksrc = static_cast<const uint8_t*>(p.k) + src0 * esz;
    d.vsrc = static_cast<const uint8_t*>(p.v) + src0 * esz;
    d.dst = p.data + (size_t)row * p.stride_bh + p.offs[mi];
    d.level = lv; d.zero_scales = 1;
    const size_t sb = (size_t)row * p.nb + blk;
    d.klo = p.klo + sb * p.G * D; d.kstep = p.kstep + sb * p.G * D;
    d.vlo = p.vlo + sb * kP * p.gv; d.vstep = p.vstep + sb * kP * p.gv;
}

template <int D>
__device__ void describe(const DemoteParams& p, int i, Desc& d) {
    clear(d);
    const int row = i / p.nb, blk = i - row * p.nb;
    const int mrow = p.per_row_meta ? row : 0;
    const size_t mi = (size_t)mrow * p.nb + blk;
    const int lo = p.level_old[mi], ln = p.level_new[mi];
    if (lo == ln || !level_ok(lo) || !level_ok(ln) || ln > lo) { d.skip = 1; return; }   // never promote
    const size_t sb = (size_t)row * p.nb + blk;
    d.src_kind = 3; d.old_level = lo;
    d.old_blk = p.data_old + (size_t)row * p.stride_old + p.offs_old[mi];
    d.klo = p.klo + sb * p.G * D; d.kstep = p.kstep + sb * p.G * D;
    d.vlo = p.vlo + sb * kP * p.gv; d.vstep = p.vstep + sb * kP * p.gv;
    d.oklo = d.klo; d.okstep = d.kstep; d.ovlo = d.vlo; d.ovstep = d.vstep;           // rewritten in place
    d.dst = p.data_new + (size_t)row * p.stride_new + p.offs_new[mi];
    d.level = ln; d.zero_scales = 1;
}

template <int D>
__device__ void describe(const PagedPackParams& p, int i, Desc& d) {
    clear(d);
    const int lv = p.level[i];
    const int64_t off = p.dst_off[i];
    if (!level_ok(lv) || off < 0) { d.skip = 1; return; }
    const size_t esz = p.src_dtype == 0 ? 4 : 2;
    d.src_kind = p.src_dtype; d.src_stride = p.token_stride;
    d.nvalid = p.nvalid ? max(1, min(p.nvalid[i], kP)) : kP;
    d.ksrc = static_cast<const uint8_t*>(p.k) + (size_t)p.src_off[i] * esz;
    d.vsrc = static_cast<const uint8_t*>(p.v) + (size_t)p.src_off[i] * esz;
    d.dst = p.pool + off; d.level = lv;
    d.ek = p.ek ? p.ek + i : nullptr; d.ev = p.ev ? p.ev + i : nullptr;
    const __half *a, *b, *c, *e;
    scales_behind(d.dst, lv, D, p.G, p.gv, a, b, c, e);
    d.klo = const_cast<__half*>(a); d.kstep = const_cast<__half*>(b);
    d.vlo = const_cast<__half*>(c); d.vstep = const_cast<__half*>(e);
}

template <int D>
__device__ void describe(const PagedDemoteParams& p, int i, Desc& d) {
    clear(d);
    const int lo = p.level_old[i], ln = p.level_new[i];
    const int64_t oo = p.off_old[i], on = p.off_new[i];
    if (lo == ln || !level_ok(lo) || !level_ok(ln) || ln > lo || oo < 0 || on < 0) { d.skip = 1; return; }
    d.src_kind = 3; d.old_level = lo; d.old_blk = p.pool_old + oo;
    scales_behind(d.old_blk, lo, D, p.G, p.gv, d.oklo, d.okstep, d.ovlo, d.ovstep);
    d.dst = p.pool_new + on; d.level = ln;
    d.ek = p.ek ? p.ek + i : nullptr; d.ev = p.ev ? p.ev + i : nullptr;
    const __half *a, *b, *c, *e;
    scales_behind(d.dst, ln, D, p.G, p.gv, a, b, c, e);
    d.klo = const_cast<__half*>(a); d.kstep = const_cast<__half*>(b);
    d.vlo = const_cast<__half*>(c); d.vstep = const_cast<__half*>(e);
}

// The producer lane: look block i up and start its copies into a stage; a source the copy engine cannot take
// (a token stride other than D, an address that is not 16-byte aligned) is left for the working threads to
// copy by hand when the block's turn comes.
template <int D, class P>
__device__ void fetch(const P& p, int i, int n, Smem& sm, int s, int G, int gv) {
    Desc d;
    if (i >= n) { clear(d); d.skip = 2; sm.desc[s] = d; bar_arrive(&sm.full[s]); return; }
    describe<D>(p, i, d);
    uint8_t* st = sm.stage[s];
    if (!d.skip) {
        if (d.src_kind != 3 && d.src_stride == D && al16(d.ksrc) && al16(d.vsrc)) {
            const uint32_t bytes = (uint32_t)d.nvalid * D * 2;
            d.staged = 1;
            sm.desc[s] = d;
            bar_expect(&sm.full[s], 2 * bytes);
            bulk(st, d.ksrc, bytes, &sm.full[s]);
            bulk(st + kP * D * 2, d.vsrc, bytes, &sm.full[s]);
            return;
        }
        if (d.src_kind == 3) {
            const bool q = d.old_level == 8 || d.old_level == 4 || d.old_level == 2;
            const uint32_t bytes = 2u * (uint32_t)half_bytes(d.old_level, D), ks = (uint32_t)G * D * 2, vs = (uint32_t)kP * gv * 2;
            if (al16(d.old_blk) && (!q || (al16(d.oklo) && al16(d.okstep) && al16(d.ovlo) && al16(d.ovstep) && ks % 16 == 0 && vs % 16 == 0))) {
                d.staged = 1;
                sm.desc[s] = d;
                bar_expect(&sm.full[s], bytes + (q ? 2 * ks + 2 * vs : 0u));
                bulk(st, d.old_blk, bytes, &sm.full[s]);
                if (q) {
                    uint8_t* sc = st + kTileBytes;
                    bulk(sc, d.oklo, ks, &sm.full[s]);
                    bulk(sc + ks, d.okstep, ks, &sm.full[s]);
                    bulk(sc + 2 * ks, d.ovlo, vs, &sm.full[s]);
                    bulk(sc + 2 * ks + vs, d.ovstep, vs, &sm.full[s]);
                }
                return;
            }
        }
    }
    sm.desc[s] = d;
    bar_arrive(&sm.full[s]);
}

// All threads: bring a block the copy engine could not take into the stage, in the same layout.
template <int D>
__device__ void copy_by_hand(const Desc& d, uint8_t* st, int G, int gv) {
    const int tid = threadIdx.x;
    if (d.src_kind != 3) {
        const uint16_t* ks = static_cast<const uint16_t*>(d.ksrc);
        const uint16_t* vs = static_cast<const uint16_t*>(d.vsrc);
        uint16_t* kd = reinterpret_cast<uint16_t*>(st);
        uint16_t* vd = kd + kP * D;
        for (int e = tid; e < d.nvalid * D; e += rq::kThreads) {
            const int t = e / D, c = e - t * D;
            kd[e] = ks[(size_t)t * d.src_stride + c];
            vd[e] = vs[(size_t)t * d.src_stride + c];
        }
        return;
    }
    const int bytes = 2 * half_bytes(d.old_level, D);
    for (int e = tid; e < bytes; e += rq::kThreads) st[e] = d.old_blk[e];
    if (d.old_level == 8 || d.old_level == 4 || d.old_level == 2) {
        __half* sc = reinterpret_cast<__half*>(st + kTileBytes);
        for (int e = tid; e < G * D; e += rq::kThreads) { sc[e] = d.oklo[e]; sc[G * D + e] = d.okstep[e]; }
        for (int e = tid; e < kP * gv; e += rq::kThreads) { sc[2 * G * D + e] = d.ovlo[e]; sc[2 * G * D + kP * gv + e] = d.ovstep[e]; }
    }
}

constexpr int kStagedThreads = rq::kThreads + 32;      // 256 working threads + the producer warp

template <int D, class P>
__global__ void __launch_bounds__(kStagedThreads, 2) staged_kernel(P p, int n, int group) {
    extern __shared__ __align__(128) uint8_t raw[];
    Smem& sm = *reinterpret_cast<Smem*>(raw);
    const int tid = threadIdx.x;
    const int kg = min(group, kP), vg = min(group, D);
    const int G = kP / kg, gv = D / vg;
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) { bar_init(&sm.full[s], 1); bar_init(&sm.empty[s], 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (tid >= rq::kThreads) {
        // ---- producer warp (one lane): looks blocks up and starts their copies, a stage ahead of the
        // workers, so that neither the table look-ups nor the copies are ever waited for by them
        if (tid == rq::kThreads) {
            for (int it = 0;; ++it) {
                const int s = it % kStages;
                if (it >= kStages && !bar_wait(&sm.empty[s], (uint32_t)(it / kStages - 1) & 1u)) {
                    atomicExch(&g_status, 1);          // the workers never released the stage
                    return;
                }
                const int i = (int)blockIdx.x + it * (int)gridDim.x;
                fetch<D>(p, i, n, sm, s, G, gv);
                if (i >= n) return;
            }
        }
        return;
    }
    for (int it = 0;; ++it) {
        const int s = it % kStages;
        const bool ok = bar_wait(&sm.full[s], (uint32_t)(it / kStages) & 1u);
        uint32_t all_ok;
        asm volatile("{ .reg .pred p, q; setp.ne.u32 q, %1, 0; bar.red.and.pred p, 1, 256, q; selp.u32 %0, 1, 0, p; }"
                     : "=r"(all_ok) : "r"((uint32_t)ok) : "memory");
        if (!all_ok) {                                 // a copy never landed: flag it and stop
            if (tid == 0) atomicExch(&g_status, 1);
            return;
        }
        const Desc& d = sm.desc[s];
        if (d.skip == 2) return;                       // past the last block
        if (!d.skip) {
            uint8_t* st = sm.stage[s];
            if (!d.staged) {
                copy_by_hand<D>(d, st, G, gv);
                rq::work_sync();
            }
            rq::Job j;
            j.src_kind = 0; j.ksrc = j.vsrc = nullptr; j.src_stride = 0; j.nvalid = kP; j.old_blk = nullptr; j.old_level = 0;
            j.oklo = j.okstep = j.ovlo = j.ovstep = nullptr;
            j.dst = d.dst; j.level = d.level; j.klo = d.klo; j.kstep = d.kstep; j.vlo = d.vlo; j.vstep = d.vstep;
            j.zero_scales = d.zero_scales; j.ek = d.ek; j.ev = d.ev; j.group = group;
            rq::StagedSrc src;
            src.kgs = 31 - __clz(kg); src.vgs = 31 - __clz(vg); src.k = st; src.nvalid = d.nvalid; src.level = d.old_level;
            if (d.src_kind != 3 || d.old_level == 16) {        // a rung-16 block is two bf16 tiles like dense rows
                src.kind = d.src_kind == 2 ? 2 : 1;
                src.v = st + kP * D * 2;
            } else {
                src.kind = 3;
                src.v = st + half_bytes(d.old_level, D);
            }
            src.klo = reinterpret_cast<const __half*>(st + kTileBytes); src.kstep = src.klo + G * D;
            src.vlo = src.kstep + G * D; src.vstep = src.vlo + kP * gv;
            rq::requantise_staged<D>(src, j, sm.work);
        }
        rq::work_sync();                               // every worker is done with the stage and the work area
        if (tid == 0) bar_arrive(&sm.empty[s]);
    }
}

// fp32 rows do not fit the stages: one CTA per block, straight from global memory.
template <int D, class P>
__global__ void __launch_bounds__(rq::kThreads, 2) direct_kernel(P p, int group) {
    __shared__ rq::Shared sm;
    Desc d;
    describe<D>(p, (int)blockIdx.x, d);
    if (d.skip) return;
    rq::Job j;
    j.src_kind = d.src_kind; j.ksrc = d.ksrc; j.vsrc = d.vsrc; j.src_stride = d.src_stride; j.nvalid = d.nvalid;
    j.old_blk = d.old_blk; j.old_level = d.old_level; j.oklo = d.oklo; j.okstep = d.okstep; j.ovlo = d.ovlo; j.ovstep = d.ovstep;
    j.dst = d.dst; j.level = d.level; j.klo = d.klo; j.kstep = d.kstep; j.vlo = d.vlo; j.vstep = d.vstep;
    j.zero_scales = d.zero_scales; j.ek = d.ek; j.ev = d.ev; j.group = group;
    rq::requantise<D, false>(j, sm);
}

template <int D, class P>
static int launch(const P& p, int n, int group, bool fp32_rows, cudaStream_t stream) {
    if (fp32_rows) {
        direct_kernel<D, P><<<n, rq::kThreads, 0, stream>>>(p, group);
        GKV_LAUNCH_CHECK();
        return GKV_OK;
    }
    int dev = 0, sms = 0;
    GKV_CUDA_TRY(cudaGetDevice(&dev));
    GKV_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    GKV_CUDA_TRY(cudaFuncSetAttribute(staged_kernel<D, P>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)));
    const int grid = n < 2 * sms ? n : 2 * sms;
    staged_kernel<D, P><<<grid, kStagedThreads, sizeof(Smem), stream>>>(p, n, group);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

template <class P>
static int launch_d(const P& p, int n, int D, int group, bool fp32_rows, cudaStream_t stream) {
    return D == 128 ? launch<128, P>(p, n, group, fp32_rows, stream) : launch<64, P>(p, n, group, fp32_rows, stream);
}

}  // namespace st

static size_t tile_smem(int D) { return (size_t)kP * (2 * tile_ld(D) * sizeof(float) + D); }

static int set_smem(const void* fn, size_t bytes) {
    GKV_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return GKV_OK;
}

}  // namespace gkv

extern "C" {

int gkv_pack_blocks(const void* k, const void* v, int src_dtype, uint8_t* data, const int64_t* offs,
                    void* klo, void* kstep, void* vlo, void* vstep, const int32_t* level,
                    const int32_t* valid, int rows, int nb, int b_lo, int b_hi, int D, int block,
                    int group, int64_t stride_bh, int meta_rows, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (rows <= 0 || nb <= 0 || D <= 0 || D > kMaxD || D % 8 || group <= 0) return GKV_E_SHAPE;
    if (kP % min(group, kP) || D % min(group, D)) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (b_lo < 0 || b_hi > nb || b_lo > b_hi || src_dtype < 0 || src_dtype > 2) return GKV_E_ARG;
    if (!k || !v || !data || !offs || !klo || !kstep || !vlo || !vstep || !level) return GKV_E_NULL;
    if (b_lo == b_hi) return GKV_OK;
    PackParams p;
    p.k = k; p.v = v; p.src_dtype = src_dtype; p.data = data; p.offs = offs;
    p.klo = (__half*)klo; p.kstep = (__half*)kstep; p.vlo = (__half*)vlo; p.vstep = (__half*)vstep;
    p.level = level; p.valid = valid; p.nb = nb; p.b_lo = b_lo; p.D = D; p.group = group;
    p.G = (kP + group - 1) / group; p.gv = (D + group - 1) / group; p.per_row_meta = meta_rows != 1;
    p.stride_bh = stride_bh;
    p.nbx = b_hi - b_lo;
    if (rq::shape_ok(D, group)) return st::launch_d(p, rows * (b_hi - b_lo), D, group, src_dtype == 0, (cudaStream_t)stream);
    int rc = set_smem((const void*)pack_blocks_kernel, tile_smem(kMaxD));
    if (rc) return rc;
    pack_blocks_kernel<<<dim3(b_hi - b_lo, rows), kPackThreads, tile_smem(D), (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

int gkv_demote_blocks(const uint8_t* data_old, const int64_t* offs_old, const int32_t* level_old,
                      uint8_t* data_new, const int64_t* offs_new, const int32_t* level_new, void* klo,
                      void* kstep, void* vlo, void* vstep, int rows, int nb, int D, int block, int group,
                      int64_t stride_old, int64_t stride_new, int meta_rows, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (rows <= 0 || nb <= 0 || D <= 0 || D > kMaxD || D % 8 || group <= 0) return GKV_E_SHAPE;
    if (kP % min(group, kP) || D % min(group, D)) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (!data_old || !offs_old || !level_old || !data_new || !offs_new || !level_new || !klo || !kstep ||
        !vlo || !vstep)
        return GKV_E_NULL;
    DemoteParams p;
    p.data_old = data_old; p.offs_old = offs_old; p.level_old = level_old;
    p.data_new = data_new; p.offs_new = offs_new; p.level_new = level_new;
    p.klo = (__half*)klo; p.kstep = (__half*)kstep; p.vlo = (__half*)vlo; p.vstep = (__half*)vstep;
    p.nb = nb; p.D = D; p.group = group; p.G = (kP + group - 1) / group; p.gv = (D + group - 1) / group;
    p.per_row_meta = meta_rows != 1; p.stride_old = stride_old; p.stride_new = stride_new;
    if (rq::shape_ok(D, group)) return st::launch_d(p, rows * nb, D, group, false, (cudaStream_t)stream);
    int rc = set_smem((const void*)demote_blocks_kernel, tile_smem(kMaxD));
    if (rc) return rc;
    demote_blocks_kernel<<<dim3(nb, rows), kPackThreads, tile_smem(D), (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

int gkv_unpack_blocks(const uint8_t* data, const int64_t* offs, const void* klo, const void* kstep,
                      const void* vlo, const void* vstep, const int32_t* level, float* k_out, float* v_out,
                      int rows, int nb, int D, int block, int group, int64_t stride_bh, int meta_rows,
                      void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (rows <= 0 || nb <= 0 || D <= 0 || D > kMaxD || group <= 0) return GKV_E_SHAPE;
    if (meta_rows != 1 && meta_rows != rows) return GKV_E_SHAPE;
    if (!data || !offs || !klo || !kstep || !vlo || !vstep || !level || !k_out || !v_out) return GKV_E_NULL;
    UnpackParams p;
    p.data = data; p.offs = offs;
    p.klo = (const __half*)klo; p.kstep = (const __half*)kstep; p.vlo = (const __half*)vlo; p.vstep = (const __half*)vstep;
    p.level = level; p.k_out = k_out; p.v_out = v_out; p.nb = nb; p.D = D; p.group = group;
    p.G = (kP + group - 1) / group; p.gv = (D + group - 1) / group; p.per_row_meta = meta_rows != 1;
    p.stride_bh = stride_bh;
    unpack_blocks_kernel<<<dim3(nb, rows), kPackThreads, 0, (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

size_t gkv_paged_block_bytes(int level, int D, int group) {
    using namespace gkv;
    if (!level_ok(level) || D <= 0 || group <= 0) return 0;
    const int kg = group < kP ? group : kP, vg = group < D ? group : D;
    const size_t scales = (level == 8 || level == 4 || level == 2) ? (size_t)4 * ((size_t)(kP / kg) * D + (size_t)kP * (D / vg)) : 0;
    return (size_t)2 * half_bytes(level, D) + scales;
}

int gkv_paged_pack_blocks(const void* k, const void* v, int src_dtype, const int64_t* src_off, int64_t token_stride,
                          const int32_t* nvalid, uint8_t* pool, const int64_t* dst_off, const int32_t* level,
                          float* ek, float* ev, int n, int D, int block, int group, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (n < 0 || !rq::shape_ok(D, group) || token_stride < D) return GKV_E_SHAPE;
    if (src_dtype < 0 || src_dtype > 2 || (ek == nullptr) != (ev == nullptr)) return GKV_E_ARG;
    if (n == 0) return GKV_OK;
    if (!k || !v || !src_off || !pool || !dst_off || !level) return GKV_E_NULL;
    PagedPackParams p;
    p.k = k; p.v = v; p.src_dtype = src_dtype; p.src_off = src_off; p.token_stride = token_stride; p.nvalid = nvalid;
    p.pool = pool; p.dst_off = dst_off; p.level = level; p.ek = ek; p.ev = ev; p.group = group;
    p.G = kP / min(group, kP); p.gv = D / min(group, D);
    return st::launch_d(p, n, D, group, src_dtype == 0, (cudaStream_t)stream);
}

int gkv_paged_demote_blocks(const uint8_t* pool_old, const int64_t* off_old, const int32_t* level_old,
                            uint8_t* pool_new, const int64_t* off_new, const int32_t* level_new, float* ek,
                            float* ev, int n, int D, int block, int group, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (n < 0 || !rq::shape_ok(D, group)) return GKV_E_SHAPE;
    if ((ek == nullptr) != (ev == nullptr)) return GKV_E_ARG;
    if (n == 0) return GKV_OK;
    if (!pool_old || !off_old || !level_old || !pool_new || !off_new || !level_new) return GKV_E_NULL;
    PagedDemoteParams p;
    p.pool_old = pool_old; p.pool_new = pool_new; p.off_old = off_old; p.level_old = level_old;
    p.off_new = off_new; p.level_new = level_new; p.ek = ek; p.ev = ev; p.group = group;
    p.G = kP / min(group, kP); p.gv = D / min(group, D);
    return st::launch_d(p, n, D, group, false, (cudaStream_t)stream);
}

int gkv_paged_unpack_blocks(const uint8_t* pool, const int64_t* offs, const int32_t* level, float* k_out,
                            float* v_out, int n, int D, int block, int group, void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (n < 0 || !rq::shape_ok(D, group)) return GKV_E_SHAPE;
    if (n == 0) return GKV_OK;
    if (!pool || !offs || !level || !k_out || !v_out) return GKV_E_NULL;
    PagedUnpackParams p;
    p.pool = pool; p.offs = offs; p.level = level; p.k_out = k_out; p.v_out = v_out; p.D = D; p.group = group;
    p.G = kP / min(group, kP); p.gv = D / min(group, D);
    paged_unpack_kernel<<<n, kPackThreads, 0, (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

int gkv_paged_append_token(const void* k, const void* v, int src_dtype, uint8_t* pool, const int64_t* offs,
                           int32_t* valid, int32_t* lens, int32_t* status, int rows, int cap, int D, int block,
                           void* stream) {
    using namespace gkv;
    if (block != kP) return GKV_E_BLOCK;
    if (rows < 0 || cap <= 0 || D <= 0 || D > kMaxD) return GKV_E_SHAPE;
    if (src_dtype < 0 || src_dtype > 2) return GKV_E_ARG;
    if (rows == 0) return GKV_OK;
    if (!k || !v || !pool || !offs || !valid || !lens || !status) return GKV_E_NULL;
    AppendParams p;
    p.k = k; p.v = v; p.src_dtype = src_dtype; p.pool = pool; p.offs = offs; p.valid = valid; p.lens = lens;
    p.status = status; p.cap = cap; p.D = D;
    paged_append_kernel<<<rows, D <= 64 ? 64 : 128, 0, (cudaStream_t)stream>>>(p);
    GKV_LAUNCH_CHECK();
    return GKV_OK;
}

int gkv_maintenance_status(int* status_host) {
    if (!status_host) return GKV_E_NULL;
    GKV_CUDA_TRY(cudaMemcpyFromSymbol(status_host, gkv::st::g_status, sizeof(int)));
    return GKV_OK;
}

}  // extern "C"
