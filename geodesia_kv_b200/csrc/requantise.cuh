// Register-resident (re)quantisation of one 64-token block: the work of the pack and demote kernels
// for head dims 64 and 128.
//
// A CTA of 256 threads takes one block.  Thread (tr, c8) holds eight consecutive channels
// (8*c8 .. 8*c8+7) of the tokens tr, tr + ROWS, ... of K and of V — one 16-byte load per token half
// when the source is bf16/fp16 — so all of a block's global loads are in flight at once and nothing
// is staged as an fp32 tile in shared memory.  K ranges (per channel over `group` consecutive
// tokens) are reduced in the thread, across the lanes that hold the same channels, and across warps
// with integer min/max atomics on the order-preserving image of fp32 in shared memory; V ranges
// (per token over `group` consecutive channels) live inside a few neighbouring lanes.  Codes come out
// eight per thread and token, i.e. as one 8/4/2-byte store in exactly the block's byte order, and a
// warp's stores cover whole token rows.
//
// The arithmetic is the reference's (geodesia_kv/policies.py:61-77 quant_grouped, packed.py:14-44):
// step = max(hi - lo, 1e-8) / qmax in fp32, lo and step rounded to fp16, code = clamp(rint((x - lo16)
// / step16), 0, qmax) with the quotient rounded as an IEEE division rounds it, centroid = fp32 sum of
// the 64 tokens in order, divided once, rounded to fp16.
#pragma once

#include "gkv_common.cuh"

namespace gkv {
namespace rq {

constexpr int kThreads = 256;

struct Job {
    // source: dense rows (src_kind 0 fp32, 1 bf16, 2 fp16) or a packed block (src_kind 3)
    int src_kind;
    const void* ksrc;           // dense: first token row of the block
    const void* vsrc;
    int64_t src_stride;         // dense: elements between consecutive tokens
    int nvalid;                 // dense: rows beyond nvalid repeat row nvalid - 1
    const uint8_t* old_blk;     // packed source
    int old_level;
    const __half* oklo; const __half* okstep; const __half* ovlo; const __half* ovstep;
    // destination
    uint8_t* dst;
    int level;
    __half* klo; __half* kstep; __half* vlo; __half* vstep;     // written for rungs 8/4/2; zeroed for 16/1 when zero_scales
    int zero_scales;
    float* ek; float* ev;       // optional: += max over tokens of |x_t - q(x_t)|_2 for K and for V (policies.py:905-906)
    int group;
};

struct __align__(16) Shared {
    uint32_t kmin[4 * 128];     // [G][D] order-preserving keys
    uint32_t kmax[4 * 128];
    float4 ks[4 * 128];         // [G][D] (lo16, step16, 1 / step16) as fp32
    uint32_t err[2];            // max error norms (bits of non-negative floats)
    float csum[2][kP];          // centroid target: per-token squared error sums
};

__device__ __forceinline__ uint32_t fkey(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float keyf(uint32_t k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// code = clamp(rint((x - lo) / step), 0, qmax), the quotient as IEEE division rounds it: the product
// with a reciprocal is within a few ulp of it (absolute error < 1e-4 for quotients up to 255), so it
// rounds to the same integer unless it lands within 1e-3 of a tie, and only then — or when it is huge
// or not a number — is the exact division needed.
__device__ __forceinline__ uint32_t code_of(float x, float lf, float sf, float rs, float qmax) {
    // rounding to nearest-even by adding 1.5 * 2^23 (the integer then sits in the low mantissa bits) keeps
    // the work on the full-rate pipes; valid for |q| < 2^22
    constexpr float kMagic = 12582912.0f;
    const float a = __fsub_rn(x, lf);
    float q = __fmul_rn(a, rs);
    float m = __fadd_rn(q, kMagic);
    float c = __fsub_rn(m, kMagic);
    if (!(fabsf(q - c) < 0.499f) || !(fabsf(q) < 1e6f)) {
        q = __fdiv_rn(a, sf);
        c = rintf(q);
        c = (c != c) ? 0.f : fminf(fmaxf(c, 0.f), qmax);
        return (uint32_t)c;
    }
    const int ci = __float_as_int(m) - 0x4B400000;
    return (uint32_t)min(max(ci, 0), (int)qmax);
}

__device__ __forceinline__ void unpack8_16(const uint4 r, bool bf, float* out) {
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
    if (bf) {                                   // one branch for the eight values, not one per pair
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    }
}

// Eight channels (8*c8 ..) of token t of the K (which = 0) or V (which = 1) half of the source.
template <int D>
__device__ __forceinline__ void load8(const Job& j, int which, int t, int c8, float* out) {
    if (j.src_kind != 3) {
        const int ts = min(t, j.nvalid - 1);
        const size_t e = (size_t)ts * (size_t)j.src_stride + 8 * c8;
        const void* base = which ? j.vsrc : j.ksrc;
        if (j.src_kind == 0) {
            const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + e);
            if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
                const float4 a = p[0], b = p[1];
                out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
                out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) out[i] = static_cast<const float*>(base)[e + i];
            }
        } else {
            const uint16_t* p = static_cast<const uint16_t*>(base) + e;
            uint4 r;
            if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
                r = *reinterpret_cast<const uint4*>(p);
            } else {
                r.x = p[0] | ((uint32_t)p[1] << 16); r.y = p[2] | ((uint32_t)p[3] << 16);
                r.z = p[4] | ((uint32_t)p[5] << 16); r.w = p[6] | ((uint32_t)p[7] << 16);
            }
            unpack8_16(r, j.src_kind == 1, out);
        }
        return;
    }
    const int lv = j.old_level;
    const uint8_t* half = j.old_blk + (which ? half_bytes(lv, D) : 0);
    if (lv == 16) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(half) + (size_t)t * D + 8 * c8;
        uint4 r;
        if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
            r = *reinterpret_cast<const uint4*>(p);
        } else {
            r.x = p[0] | ((uint32_t)p[1] << 16); r.y = p[2] | ((uint32_t)p[3] << 16);
            r.z = p[4] | ((uint32_t)p[5] << 16); r.w = p[6] | ((uint32_t)p[7] << 16);
        }
        unpack8_16(r, true, out);
        return;
    }
    if (lv == 1) {
        const uint16_t* p = reinterpret_cast<const uint16_t*>(half) + 8 * c8;
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = half_bits_to_float(p[i]);
        return;
    }
    // eight codes = lv bytes at byte (t*D + 8*c8) * lv / 8, little-endian
    const uint8_t* cp = half + ((size_t)t * D + 8 * c8) * lv / 8;
    unsigned long long bits = 0;
    if ((reinterpret_cast<uintptr_t>(cp) & (uintptr_t)(lv - 1)) == 0) {          // lv bytes, naturally aligned
        if (lv == 8) { const uint2 r = *reinterpret_cast<const uint2*>(cp); bits = ((unsigned long long)r.y << 32) | r.x; }
        else if (lv == 4) bits = *reinterpret_cast<const uint32_t*>(cp);
        else bits = *reinterpret_cast<const uint16_t*>(cp);
    } else {
        for (int i = 0; i < lv; ++i) bits |= (unsigned long long)cp[i] << (8 * i);
    }
    const uint32_t mask = (1u << lv) - 1u;
    const int kg = min(j.group, kP), vg = min(j.group, D);
    if (which == 0) {
        const int s0 = (t / kg) * D + 8 * c8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float c = (float)((uint32_t)(bits >> (i * lv)) & mask);
            out[i] = __fmaf_rn(c, __half2float(j.okstep[s0 + i]), __half2float(j.oklo[s0 + i]));
        }
    } else {
        const int s = t * (D / vg) + (8 * c8) / vg;
        const float st = __half2float(j.ovstep[s]), lo = __half2float(j.ovlo[s]);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float c = (float)((uint32_t)(bits >> (i * lv)) & mask);
            out[i] = __fmaf_rn(c, st, lo);
        }
    }
}

// One element (token t, channel d) of the source — the centroid path walks a channel token by token.
template <int D>
__device__ __forceinline__ float load1(const Job& j, int which, int t, int d) {
    if (j.src_kind != 3) {
        const size_t e = (size_t)min(t, j.nvalid - 1) * (size_t)j.src_stride + d;
        const void* base = which ? j.vsrc : j.ksrc;
        if (j.src_kind == 0) return static_cast<const float*>(base)[e];
        const uint16_t h = static_cast<const uint16_t*>(base)[e];
        return j.src_kind == 1 ? bf16_bits_to_float(h) : half_bits_to_float(h);
    }
    const int lv = j.old_level;
    const uint8_t* half = j.old_blk + (which ? half_bytes(lv, D) : 0);
    if (lv == 16) return bf16_bits_to_float(reinterpret_cast<const uint16_t*>(half)[t * D + d]);
    if (lv == 1) return half_bits_to_float(reinterpret_cast<const uint16_t*>(half)[d]);
    const float c = (float)unpack_code(half, t * D + d, lv);
    const int kg = min(j.group, kP), vg = min(j.group, D);
    if (which == 0) {
        const int s = (t / kg) * D + d;
        return __fmaf_rn(c, __half2float(j.okstep[s]), __half2float(j.oklo[s]));
    }
    const int s = t * (D / vg) + d / vg;
    return __fmaf_rn(c, __half2float(j.ovstep[s]), __half2float(j.ovlo[s]));
}

// Eight codes of `lv` bits each -> lv bytes at `out` (byte order of the block).
__device__ __forceinline__ void store_codes(uint8_t* out, const uint32_t* c, int lv) {
    if (lv == 8) {
        const uint32_t a = c[0] | (c[1] << 8) | (c[2] << 16) | (c[3] << 24);
        const uint32_t b = c[4] | (c[5] << 8) | (c[6] << 16) | (c[7] << 24);
        if ((reinterpret_cast<uintptr_t>(out) & 7) == 0) *reinterpret_cast<uint2*>(out) = make_uint2(a, b);
        else for (int i = 0; i < 8; ++i) out[i] = (uint8_t)c[i];
    } else if (lv == 4) {
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) w |= c[i] << (4 * i);
        if ((reinterpret_cast<uintptr_t>(out) & 3) == 0) *reinterpret_cast<uint32_t*>(out) = w;
        else for (int i = 0; i < 4; ++i) out[i] = (uint8_t)(w >> (8 * i));
    } else {
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) w |= c[i] << (2 * i);
        if ((reinterpret_cast<uintptr_t>(out) & 1) == 0) *reinterpret_cast<uint16_t*>(out) = (uint16_t)w;
        else { out[0] = (uint8_t)w; out[1] = (uint8_t)(w >> 8); }
    }
}

// Shapes this path takes: D 64 or 128, group a multiple of 8 that divides 64 and D (or exceeds them).
__host__ __device__ __forceinline__ bool shape_ok(int D, int group) {
    if (D != 64 && D != 128) return false;
    const int kg = group < kP ? group : kP, vg = group < D ? group : D;
    return group % 8 == 0 && kP % kg == 0 && D % vg == 0 && kP / kg <= 4;
}

// STAGED: the source sits in shared memory (a bulk copy put it there) and is simply read again by every
// pass; otherwise the block's values are loaded once from global memory and held in registers.
template <int D, bool STAGED>
__device__ void requantise(const Job& j, Shared& sm) {
    constexpr int OPR = D / 8;                 // channel octets per token row
    constexpr int ROWS = kThreads / OPR;       // token rows the CTA covers per pass
    constexpr int NI = kP / ROWS;              // passes: tokens tr, tr + ROWS, ...
    const int tid = threadIdx.x, lane = tid & 31;
    const int c8 = tid % OPR, tr = tid / OPR;
    const int lv = j.level;
    const int kg = min(j.group, kP), vg = min(j.group, D);
    const int G = kP / kg, gv = D / vg;
    const bool quant = lv == 8 || lv == 4 || lv == 2;
    const bool radii = j.ek != nullptr;

    if (tid < 2) sm.err[tid] = 0u;
    if (quant) {
        for (int u = tid; u < G * D; u += kThreads) { sm.kmin[u] = 0xffffffffu; sm.kmax[u] = 0u; }
    } else if (j.zero_scales) {
        // the dense side tensors of the reference hold zeros for rungs 16 and 1 (pack_layout.py:25-28)
        for (int u = tid; u < G * D; u += kThreads) { j.klo[u] = __ushort_as_half(0); j.kstep[u] = __ushort_as_half(0); }
        for (int u = tid; u < kP * gv; u += kThreads) { j.vlo[u] = __ushort_as_half(0); j.vstep[u] = __ushort_as_half(0); }
    }

    if (lv == 1) {
        // centroid: thread (which, d) adds the 64 tokens of its channel in order
        float mean = 0.f;
        const int which = tid / D, d = tid - which * D;
        if (tid < 2 * D) {
            float s = 0.f;
#pragma unroll 8
            for (int t = 0; t < kP; ++t) s = __fadd_rn(s, load1<D>(j, which, t, d));
            mean = __half2float(__float2half_rn(__fdiv_rn(s, (float)kP)));
        }
        if (radii) for (int u = tid; u < 2 * kP; u += kThreads) sm.csum[u / kP][u % kP] = 0.f;
        __syncthreads();                       // every source byte has been read (the destination may overlap it)
        if (radii && tid < 2 * D) {
            for (int t = 0; t < kP; ++t) {
                const float e = __fsub_rn(load1<D>(j, which, t, d), mean);
                float s = e * e;
#pragma unroll
                for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) atomicAdd(&sm.csum[which][t], s);
            }
        }
        __syncthreads();
        if (tid < 2 * D) {
            __half* o = reinterpret_cast<__half*>(j.dst + (which ? half_bytes(1, D) : 0));
            o[d] = __float2half_rn(mean);
        }
        if (radii && tid < 2) {
            float m = 0.f;
            for (int t = 0; t < kP; ++t) m = fmaxf(m, sm.csum[tid][t]);
            float* acc = tid ? j.ev : j.ek;
            *acc += sqrtf(m);
        }
        return;
    }

    // ---- all loads first ------------------------------------------------------------------
    float kx[NI][8], vx[NI][8];
    if constexpr (!STAGED) {
#pragma unroll
        for (int i = 0; i < NI; ++i) load8<D>(j, 0, tr + i * ROWS, c8, kx[i]);
#pragma unroll
        for (int i = 0; i < NI; ++i) load8<D>(j, 1, tr + i * ROWS, c8, vx[i]);
    }
    auto values = [&](int which, int i, float* out) {
        if constexpr (STAGED) {
            load8<D>(j, which, tr + i * ROWS, c8, out);
        } else {
#pragma unroll
            for (int c = 0; c < 8; ++c) out[c] = which ? vx[i][c] : kx[i][c];
        }
    };

    if (lv == 16) {
        __syncthreads();
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            uint16_t* half = reinterpret_cast<uint16_t*>(j.dst + (w ? half_bytes(16, D) : 0));
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                float x[8];
                values(w, i, x);
                uint32_t o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const __nv_bfloat162 b = __floats2bfloat162_rn(x[2 * c], x[2 * c + 1]);
                    o[c] = *reinterpret_cast<const uint32_t*>(&b);
                }
                uint16_t* p = half + (size_t)(tr + i * ROWS) * D + 8 * c8;
                if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) *reinterpret_cast<uint4*>(p) = make_uint4(o[0], o[1], o[2], o[3]);
                else for (int c = 0; c < 4; ++c) { p[2 * c] = (uint16_t)o[c]; p[2 * c + 1] = (uint16_t)(o[c] >> 16); }
            }
        }
        return;
    }

    const float qmax = (float)((1 << lv) - 1);
    __syncthreads();                           // key tables initialised

    // ---- K ranges: thread, then the lanes with the same channels, then shared-memory atomics -------
    {
        int cur = tr / kg;
        float lo[8], hi[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) { lo[c] = INFINITY; hi[c] = -INFINITY; }
#pragma unroll
        for (int i = 0; i <= NI; ++i) {
            const int tg = i < NI ? (tr + i * ROWS) / kg : -1;
            if (tg != cur) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
#pragma unroll
                    for (int o = OPR; o < 32; o <<= 1) {
                        lo[c] = fminf(lo[c], __shfl_xor_sync(0xffffffffu, lo[c], o));
                        hi[c] = fmaxf(hi[c], __shfl_xor_sync(0xffffffffu, hi[c], o));
                    }
                    if (lane < OPR) {
                        atomicMin(&sm.kmin[cur * D + 8 * c8 + c], fkey(lo[c]));
                        atomicMax(&sm.kmax[cur * D + 8 * c8 + c], fkey(hi[c]));
                    }
                    lo[c] = INFINITY; hi[c] = -INFINITY;
                }
                cur = tg;
            }
            if (i < NI) {
                float x[8];
                values(0, i, x);
#pragma unroll
                for (int c = 0; c < 8; ++c) { lo[c] = fminf(lo[c], x[c]); hi[c] = fmaxf(hi[c], x[c]); }
            }
        }
    }
    __syncthreads();
    for (int u = tid; u < G * D; u += kThreads) {
        const float lo = keyf(sm.kmin[u]), hi = keyf(sm.kmax[u]);
        const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
        const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
        j.klo[u] = l16; j.kstep[u] = s16;
        const float sf = __half2float(s16);
        // a thread later reads the entries of its eight channels: they are laid out so that the 16 (or 8)
        // lanes of a token row read consecutive 16-byte slots
        const int tgu = u / D, du = u - tgu * D;
        sm.ks[(tgu * 8 + (du & 7)) * OPR + (du >> 3)] = make_float4(__half2float(l16), sf, __frcp_rn(sf), 0.f);
    }
    __syncthreads();                           // also: every source byte has been read before the first code is stored

    float ekmax = 0.f, evmax = 0.f;
    // ---- K codes ---------------------------------------------------------------------------
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int t = tr + i * ROWS;
        const float4* sc = sm.ks + (t / kg) * 8 * OPR + c8;
        uint32_t code[8];
        float x[8];
        values(0, i, x);
        float e2 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float4 ls = sc[c * OPR];
            code[c] = code_of(x[c], ls.x, ls.y, ls.z, qmax);
            if (radii) { const float e = x[c] - __fmaf_rn((float)code[c], ls.y, ls.x); e2 += e * e; }
        }
        store_codes(j.dst + ((size_t)t * D + 8 * c8) * lv / 8, code, lv);
        if (radii) {
#pragma unroll
            for (int o = 1; o < OPR; o <<= 1) e2 += __shfl_xor_sync(0xffffffffu, e2, o);
            ekmax = fmaxf(ekmax, e2);
        }
    }
    // ---- V: ranges inside vg/8 neighbouring lanes, scales, codes ----------------------------------
    uint8_t* vdst = j.dst + half_bytes(lv, D);
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int t = tr + i * ROWS;
        float x[8];
        values(1, i, x);
        float lo = INFINITY, hi = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; ++c) { lo = fminf(lo, x[c]); hi = fmaxf(hi, x[c]); }
        for (int o = 1; o < vg / 8; o <<= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
        const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
        const int cg = (8 * c8) / vg;
        if ((8 * c8) % vg == 0) { j.vlo[t * gv + cg] = l16; j.vstep[t * gv + cg] = s16; }
        const float lf = __half2float(l16), sf = __half2float(s16), rs = __frcp_rn(sf);
        uint32_t code[8];
        float e2 = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            code[c] = code_of(x[c], lf, sf, rs, qmax);
            if (radii) { const float e = x[c] - __fmaf_rn((float)code[c], sf, lf); e2 += e * e; }
        }
        store_codes(vdst + ((size_t)t * D + 8 * c8) * lv / 8, code, lv);
        if (radii) {
#pragma unroll
            for (int o = 1; o < OPR; o <<= 1) e2 += __shfl_xor_sync(0xffffffffu, e2, o);
            evmax = fmaxf(evmax, e2);
        }
    }
    if (radii) {
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            ekmax = fmaxf(ekmax, __shfl_xor_sync(0xffffffffu, ekmax, o));
            evmax = fmaxf(evmax, __shfl_xor_sync(0xffffffffu, evmax, o));
        }
        if (lane == 0) { atomicMax(&sm.err[0], __float_as_uint(ekmax)); atomicMax(&sm.err[1], __float_as_uint(evmax)); }
        __syncthreads();
        if (tid < 2) {
            float* acc = tid ? j.ev : j.ek;
            *acc += sqrtf(__uint_as_float(sm.err[tid]));
        }
    }
}

// ---- the same work on a block that already sits in shared memory ---------------------------------------
// Source: two 16-bit tiles [64][D] (dense bf16/fp16 rows, or a rung-16 block), or a packed block of a
// quantised rung with its four scale planes; everything 16-byte aligned.  Passes re-read the source
// instead of holding it in registers, loops over the thread's tokens are not unrolled (the whole body
// stays small enough for the instruction cache), and the rare exact division is taken once per eight
// codes, not per code.
#ifndef GKV_RQ_UNROLL
#define GKV_RQ_UNROLL 1
#endif
constexpr int kCodeUnroll = GKV_RQ_UNROLL;     // unrolling of the loops over a thread's tokens in the code passes
// The 256 working threads of a CTA meet at named barrier 1: the CTA may hold more threads (a producer
// warp that feeds the stages), which must not be part of these barriers.
__device__ __forceinline__ void work_sync() { asm volatile("bar.sync 1, 256;" ::: "memory"); }

struct StagedSrc {
    const uint8_t* k; const uint8_t* v;     // dense tiles (kind 1 bf16, 2 fp16), or the halves of the packed block (kind 3)
    int kind, nvalid, level;                // level: rung of a packed source (8, 4 or 2)
    const __half* klo; const __half* kstep; const __half* vlo; const __half* vstep;
    int kgs, vgs;                           // log2 of the K token group and of the V channel group (both powers of two)
};

template <int D>
__device__ __forceinline__ void staged8(const StagedSrc& s, int which, int t, int c8, float* out) {
    if (s.kind != 3) {
        const uint4 r = *reinterpret_cast<const uint4*>((which ? s.v : s.k) + ((size_t)min(t, s.nvalid - 1) * D + 8 * c8) * 2);
        unpack8_16(r, s.kind == 1, out);
        return;
    }
    const int lv = s.level;
    const uint8_t* cp = (which ? s.v : s.k) + ((size_t)t * D + 8 * c8) * lv / 8;
    unsigned long long bits;
    if (lv == 8) { const uint2 r = *reinterpret_cast<const uint2*>(cp); bits = ((unsigned long long)r.y << 32) | r.x; }
    else if (lv == 4) bits = *reinterpret_cast<const uint32_t*>(cp);
    else bits = *reinterpret_cast<const uint16_t*>(cp);
    const uint32_t mask = (1u << lv) - 1u;
    if (which == 0) {
        const uint4 lo4 = *reinterpret_cast<const uint4*>(s.klo + (t >> s.kgs) * D + 8 * c8);
        const uint4 st4 = *reinterpret_cast<const uint4*>(s.kstep + (t >> s.kgs) * D + 8 * c8);
        float lo[8], st[8];
        unpack8_16(lo4, false, lo);
        unpack8_16(st4, false, st);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = __fmaf_rn((float)((uint32_t)(bits >> (i * lv)) & mask), st[i], lo[i]);
    } else {
        const int si = t * (D >> s.vgs) + ((8 * c8) >> s.vgs);
        const float st = __half2float(s.vstep[si]), lo = __half2float(s.vlo[si]);
#pragma unroll
        for (int i = 0; i < 8; ++i) out[i] = __fmaf_rn((float)((uint32_t)(bits >> (i * lv)) & mask), st, lo);
    }
}

template <int D>
__device__ __forceinline__ float staged1(const StagedSrc& s, int which, int t, int d) {
    if (s.kind != 3) {
        const uint16_t h = reinterpret_cast<const uint16_t*>(which ? s.v : s.k)[(size_t)min(t, s.nvalid - 1) * D + d];
        return s.kind == 1 ? bf16_bits_to_float(h) : half_bits_to_float(h);
    }
    const float c = (float)unpack_code(which ? s.v : s.k, t * D + d, s.level);
    if (which == 0) {
        const int i = (t >> s.kgs) * D + d;
        return __fmaf_rn(c, __half2float(s.kstep[i]), __half2float(s.klo[i]));
    }
    const int i = t * (D >> s.vgs) + (d >> s.vgs);
    return __fmaf_rn(c, __half2float(s.vstep[i]), __half2float(s.vlo[i]));
}

// Eight codes at once.  The fast path takes the quotient as a product with the reciprocal of the step:
// that is within |q| * 2^-22 of the correctly rounded division, so both round to the same integer
// unless the product lands that close to a tie.  `tie` = 0.5 minus several times that bound for the
// rung's largest quotient; only codes that fail the test (or are not numbers) are redone with the
// IEEE division, one by one — a warp rarely has any.
__device__ __forceinline__ float max_nan(float a, float b) {      // maximum that keeps a NaN operand
    float d;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(d) : "f"(a), "f"(b));
    return d;
}

__device__ __forceinline__ void codes8(const float* x, const float* lf, const float* sf, const float* rs, float qmax, int qmaxi,
                                       float tie, uint32_t* code) {
    constexpr float kMagic = 12582912.0f;      // 1.5 * 2^23: adding it rounds to nearest-even into the low mantissa bits
    float worst = 0.f;                         // largest distance of a quotient from the integer it rounded to (NaN sticks)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const float q = __fmul_rn(__fsub_rn(x[c], lf[c]), rs[c]);
        const float m = __fadd_rn(q, kMagic);
        worst = max_nan(worst, fabsf(q - __fsub_rn(m, kMagic)));
        code[c] = (uint32_t)min(max(__float_as_int(m) - 0x4B400000, 0), qmaxi);   // out-of-range q clamps correctly
    }
    if (!(worst < tie)) {                      // some quotient is near a tie or not a number: redo those exactly
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float a = __fsub_rn(x[c], lf[c]);
            const float q0 = __fmul_rn(a, rs[c]);
            if (!(fabsf(q0 - rintf(q0)) < tie)) {
                const float q = __fdiv_rn(a, sf[c]);
                float r = rintf(q);
                r = (r != r) ? 0.f : fminf(fmaxf(r, 0.f), qmax);
                code[c] = (uint32_t)r;
            }
        }
    }
}

template <int D, int LV>
__device__ __forceinline__ void quantise_staged(const StagedSrc& src, const Job& j, Shared& sm) {
    constexpr int OPR = D / 8, ROWS = kThreads / OPR, NI = kP / ROWS;
    constexpr int lv = LV;
    const int tid = threadIdx.x, lane = tid & 31;
    const int c8 = tid % OPR, tr = tid / OPR;
    const int kgs = src.kgs, vgs = src.vgs, vg = 1 << vgs;
    const int G = kP >> kgs, gv = D >> vgs;
    const bool radii = j.ek != nullptr;
    const float qmax = (float)((1 << lv) - 1);
    const int qmaxi = (1 << lv) - 1;
    const float tie = 0.5f - (qmax + 1.0f) * 1e-6f;
    work_sync();                           // key tables initialised

    // ---- K ranges: thread, then the lanes with the same channels, then shared-memory atomics -------
    {
        int cur = tr >> kgs;
        float lo[8], hi[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) { lo[c] = INFINITY; hi[c] = -INFINITY; }
#pragma unroll
        for (int i = 0; i <= NI; ++i) {
            const int tg = i < NI ? (tr + i * ROWS) >> kgs : -1;
            if (tg != cur) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
#pragma unroll
                    for (int o = OPR; o < 32; o <<= 1) {
                        lo[c] = fminf(lo[c], __shfl_xor_sync(0xffffffffu, lo[c], o));
                        hi[c] = fmaxf(hi[c], __shfl_xor_sync(0xffffffffu, hi[c], o));
                    }
                    if (lane < OPR) {
                        atomicMin(&sm.kmin[cur * D + 8 * c8 + c], fkey(lo[c]));
                        atomicMax(&sm.kmax[cur * D + 8 * c8 + c], fkey(hi[c]));
                    }
                    lo[c] = INFINITY; hi[c] = -INFINITY;
                }
                cur = tg;
            }
            if (i < NI) {
                float x[8];
                staged8<D>(src, 0, tr + i * ROWS, c8, x);
#pragma unroll
                for (int c = 0; c < 8; ++c) { lo[c] = fminf(lo[c], x[c]); hi[c] = fmaxf(hi[c], x[c]); }
            }
        }
    }
    float ekmax = 0.f, evmax = 0.f;
    // ---- V: ranges inside vg/8 neighbouring lanes, scales, codes — done here, between the K range atomics and
    // the barrier that publishes them, so that warps which finish early have work instead of a wait
    uint8_t* vdst = j.dst + half_bytes(lv, D);
#pragma unroll kCodeUnroll
    for (int i = 0; i < NI; ++i) {
        const int t = tr + i * ROWS;
        float x[8];
        staged8<D>(src, 1, t, c8, x);
        float lo = INFINITY, hi = -INFINITY;
#pragma unroll
        for (int c = 0; c < 8; ++c) { lo = fminf(lo, x[c]); hi = fmaxf(hi, x[c]); }
        for (int o = 1; o < vg / 8; o <<= 1) {
            lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
            hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
        }
        const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
        const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
        const int cg = (8 * c8) >> vgs;
        if (((8 * c8) & (vg - 1)) == 0) { j.vlo[t * gv + cg] = l16; j.vstep[t * gv + cg] = s16; }
        const float l1 = __half2float(l16), s1 = __half2float(s16), r1 = __frcp_rn(s1);
        float lf[8], sf[8], rs[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) { lf[c] = l1; sf[c] = s1; rs[c] = r1; }
        uint32_t code[8];
        codes8(x, lf, sf, rs, qmax, qmaxi, tie, code);
        store_codes(vdst + ((size_t)t * D + 8 * c8) * lv / 8, code, lv);
        if (radii) {
            float e2 = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) { const float e = x[c] - __fmaf_rn((float)code[c], s1, l1); e2 += e * e; }
#pragma unroll
            for (int o = 1; o < OPR; o <<= 1) e2 += __shfl_xor_sync(0xffffffffu, e2, o);
            evmax = fmaxf(evmax, e2);
        }
    }
    work_sync();
    for (int u = tid; u < G * D; u += kThreads) {
        const float lo = keyf(sm.kmin[u]), hi = keyf(sm.kmax[u]);
        const float step = __fdiv_rn(fmaxf(__fsub_rn(hi, lo), 1e-8f), qmax);
        const __half l16 = __float2half_rn(lo), s16 = __float2half_rn(step);
        j.klo[u] = l16; j.kstep[u] = s16;
        const float sf = __half2float(s16);
        const int tgu = u / D, du = u - tgu * D;
        sm.ks[(tgu * 8 + (du & 7)) * OPR + (du >> 3)] = make_float4(__half2float(l16), sf, __frcp_rn(sf), 0.f);
    }
    work_sync();

    // ---- K codes ---------------------------------------------------------------------------
#pragma unroll kCodeUnroll
    for (int i = 0; i < NI; ++i) {
        const int t = tr + i * ROWS;
        const float4* sc = sm.ks + (t >> kgs) * 8 * OPR + c8;
        float x[8], lf[8], sf[8], rs[8];
        staged8<D>(src, 0, t, c8, x);
#pragma unroll
        for (int c = 0; c < 8; ++c) { const float4 ls = sc[c * OPR]; lf[c] = ls.x; sf[c] = ls.y; rs[c] = ls.z; }
        uint32_t code[8];
        codes8(x, lf, sf, rs, qmax, qmaxi, tie, code);
        store_codes(j.dst + ((size_t)t * D + 8 * c8) * lv / 8, code, lv);
        if (radii) {
            float e2 = 0.f;
#pragma unroll
            for (int c = 0; c < 8; ++c) { const float e = x[c] - __fmaf_rn((float)code[c], sf[c], lf[c]); e2 += e * e; }
#pragma unroll
            for (int o = 1; o < OPR; o <<= 1) e2 += __shfl_xor_sync(0xffffffffu, e2, o);
            ekmax = fmaxf(ekmax, e2);
        }
    }
    if (radii) {
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            ekmax = fmaxf(ekmax, __shfl_xor_sync(0xffffffffu, ekmax, o));
            evmax = fmaxf(evmax, __shfl_xor_sync(0xffffffffu, evmax, o));
        }
        if (lane == 0) { atomicMax(&sm.err[0], __float_as_uint(ekmax)); atomicMax(&sm.err[1], __float_as_uint(evmax)); }
        work_sync();
        if (tid < 2) {
            float* acc = tid ? j.ev : j.ek;
            *acc += sqrtf(__uint_as_float(sm.err[tid]));
        }
    }
}

template <int D>
__device__ void requantise_staged(const StagedSrc& src, const Job& j, Shared& sm) {
    constexpr int OPR = D / 8, ROWS = kThreads / OPR, NI = kP / ROWS;
    const int tid = threadIdx.x, lane = tid & 31;
    const int c8 = tid % OPR, tr = tid / OPR;
    const int lv = j.level;
    const int kgs = src.kgs, vgs = src.vgs, vg = 1 << vgs;
    const int G = kP >> kgs, gv = D >> vgs;
    const bool quant = lv == 8 || lv == 4 || lv == 2;
    const bool radii = j.ek != nullptr;

    if (tid < 2) sm.err[tid] = 0u;
    if (quant) {
        for (int u = tid; u < G * D; u += kThreads) { sm.kmin[u] = 0xffffffffu; sm.kmax[u] = 0u; }
    } else if (j.zero_scales) {
        for (int u = tid; u < G * D; u += kThreads) { j.klo[u] = __ushort_as_half(0); j.kstep[u] = __ushort_as_half(0); }
        for (int u = tid; u < kP * gv; u += kThreads) { j.vlo[u] = __ushort_as_half(0); j.vstep[u] = __ushort_as_half(0); }
    }

    if (lv == 1) {
        // centroid: thread (which, d) adds the 64 tokens of its channel in order
        const int which = tid / D, d = tid - which * D;
        float mean = 0.f;
        if (tid < 2 * D) {
            float s = 0.f;
#pragma unroll 8
            for (int t = 0; t < kP; ++t) s = __fadd_rn(s, staged1<D>(src, which, t, d));
            mean = __half2float(__float2half_rn(__fdiv_rn(s, (float)kP)));
            reinterpret_cast<__half*>(j.dst + (which ? half_bytes(1, D) : 0))[d] = __float2half_rn(mean);
        }
        if (radii) {
            for (int u = tid; u < 2 * kP; u += kThreads) sm.csum[u / kP][u % kP] = 0.f;
            work_sync();
            if (tid < 2 * D) {
                for (int t = 0; t < kP; ++t) {
                    const float e = __fsub_rn(staged1<D>(src, which, t, d), mean);
                    float s2 = e * e;
#pragma unroll
                    for (int o = 16; o; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
                    if (lane == 0) atomicAdd(&sm.csum[which][t], s2);
                }
            }
            work_sync();
            if (tid < 2) {
                float m = 0.f;
                for (int t = 0; t < kP; ++t) m = fmaxf(m, sm.csum[tid][t]);
                float* acc = tid ? j.ev : j.ek;
                *acc += sqrtf(m);
            }
        }
        return;
    }

    if (lv == 16) {
#pragma unroll
        for (int w = 0; w < 2; ++w) {
            uint16_t* half = reinterpret_cast<uint16_t*>(j.dst + (w ? half_bytes(16, D) : 0));
#pragma unroll
            for (int i = 0; i < NI; ++i) {
                float x[8];
                staged8<D>(src, w, tr + i * ROWS, c8, x);
                uint32_t o[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const __nv_bfloat162 b = __floats2bfloat162_rn(x[2 * c], x[2 * c + 1]);
                    o[c] = *reinterpret_cast<const uint32_t*>(&b);
                }
                uint16_t* p = half + (size_t)(tr + i * ROWS) * D + 8 * c8;
                if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) *reinterpret_cast<uint4*>(p) = make_uint4(o[0], o[1], o[2], o[3]);
                else for (int c = 0; c < 4; ++c) { p[2 * c] = (uint16_t)o[c]; p[2 * c + 1] = (uint16_t)(o[c] >> 16); }
            }
        }
        return;
    }

    // the quantised rungs: one body per rung, so that every shift, mask and byte offset is a constant
    if (lv == 8) quantise_staged<D, 8>(src, j, sm);
    else if (lv == 4) quantise_staged<D, 4>(src, j, sm);
    else quantise_staged<D, 2>(src, j, sm);
}


}  // namespace rq
}  // namespace gkv
