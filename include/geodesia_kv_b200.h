/*
 * geodesia_kv_b200 — C ABI of the B200 (sm_100a) packed-KV decode path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its
 * comment says "host".  Every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*), never synchronises, allocates no device memory (the caller
 * passes the workspace) and returns 0 or a negative GKV_E_* code; launch errors
 * are returned as GKV_E_CUDA and the CUDA error stays readable through
 * gkv_last_cuda_error().  The library has no global state besides that code.
 *
 * Each entry point names the interface of geodesia-ai/geodesia-kv it replaces.
 *
 * Packed block format (the reference's; geodesia_kv/pack_layout.py:29-45 and
 * geodesia_kv_cuda/mixed_attn.cu:93-159).  A cache row (one batch entry, one KV
 * head) is a byte string; block b starts at byte offs[b] and holds K then V:
 *   level 16      P*D bf16 each, row major [token][channel]
 *   level 8/4/2   P*D codes each, code i = token*D + channel in byte i/(8/bits)
 *                 at bit (i % (8/bits))*bits; value = code*step + lo in fp32 with
 *                 fp16 scales: K scales (nb, G, D) indexed [token/g][channel],
 *                 V scales (nb, P, gv) indexed [token][channel/g]
 *   level 1       D fp16 each: one centroid standing for all valid tokens
 * P = 64 tokens per block, G = ceil(P/g), gv = ceil(D/g).
 */
#ifndef GEODESIA_KV_B200_H
#define GEODESIA_KV_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GKV_OK 0
#define GKV_E_BLOCK (-1)     /* block size other than 64 (mixed_attn.cu:219)            */
#define GKV_E_SHAPE (-2)     /* unsupported or inconsistent shape                         */
#define GKV_E_NULL (-3)      /* a required pointer is null                                */
#define GKV_E_WORKSPACE (-4) /* workspace missing, misaligned or too small                */
#define GKV_E_CUDA (-5)      /* a CUDA call failed; see gkv_last_cuda_error()             */
#define GKV_E_ARG (-6)       /* an argument is out of range                               */
#define GKV_E_STATIC_SCRATCH (-7) /* gkv_mixed_attn_decode_static: problem exceeds the built-in scratch */

int gkv_abi_version(void);
const char *gkv_error_string(int code); /* host string, static storage */
int gkv_last_cuda_error(void);          /* cudaError_t of the last failing CUDA call, 0 if none */

/* ---- decode attention ------------------------------------------------------
 * Replaces mixed_attn_decode, geodesia_kv_cuda/mixed_attn.cu:202-244 (host),
 * :44-167 (slice kernel), :171-200 (combine), bound by binding.cpp:10-13.
 *
 *   q        (B, Hq, D) fp32, already multiplied by the softmax scale
 *   data     (B, Hkv, stride_bh) bytes
 *   offs     int64, level/valid int32: nb entries per metadata row;
 *            meta_rows = 1 shares one row over every (b, hkv) — the reference's
 *            convention — and meta_rows = B*Hkv gives each cache row its own
 *   klo,kstep (B, Hkv, nb, G, D) fp16;  vlo,vstep (B, Hkv, nb, P, gv) fp16
 *   out      (B, Hq, D) fp32
 * Query head h attends over cache row h / (Hq/Hkv): Hq == Hkv is the
 * reference's one-query-per-row call, Hq > Hkv reads each row once for the
 * whole GQA group.  Tokens j >= valid[b] are masked.  `block` must be 64.
 * Scratch: gkv_decode_workspace_bytes() bytes, 256-byte aligned, private to
 * the call until it completes on `stream`.
 */
size_t gkv_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int nb);

/* Number of kernels one decode call of this shape launches (host arithmetic only; for callers
 * that account for launches, e.g. a benchmark).  Assumes 16-byte aligned scale planes, which is
 * what selects the tensor-core kernel.  No counterpart in the reference.                       */
int gkv_decode_kernel_launches(int B, int Hq, int Hkv, int D, int nb, int group);

int gkv_mixed_attn_decode(const float *q, const uint8_t *data, const int64_t *offs,
                          const void *klo, const void *kstep, const void *vlo, const void *vstep,
                          const int32_t *level, const int32_t *valid, float *out,
                          void *workspace, size_t workspace_bytes,
                          int B, int Hq, int Hkv, int D, int nb, int block, int group,
                          int64_t stride_bh, int meta_rows, void *stream);

/* Same attention, but stops before the normalisation: writes, per (b, hq),
 * D+2 floats  [m, l, o[0..D)]  with o = sum_j exp(s_j - m) v_j  — the merged
 * state of mixed_attn.cu:161-166 over the whole row.  Used when a sequence is
 * split over several GPUs: each rank runs this on its blocks, the (m, l, o)
 * records are all-gathered and gkv_combine_partials() finishes the softmax.
 */
int gkv_mixed_attn_decode_partial(const float *q, const uint8_t *data, const int64_t *offs,
                                  const void *klo, const void *kstep, const void *vlo, const void *vstep,
                                  const int32_t *level, const int32_t *valid, float *partial,
                                  void *workspace, size_t workspace_bytes,
                                  int B, int Hq, int Hkv, int D, int nb, int block, int group,
                                  int64_t stride_bh, int meta_rows, void *stream);

/* Decode attention for callers that cannot allocate device memory.  It has no counterpart in
 * the reference: the reference's launcher allocates its split buffers through torch on every call.
 * Some hosts of this library cannot do that — a serving loop that has handed all of HBM to its
 * own pool, a plugin called from inside a region where the CUDA allocator must not be entered,
 * a runtime without torch at all — and gkv_mixed_attn_decode still asks them for a workspace.
 * This variant takes none: its split records and work counter live in a fixed array inside the
 * library image (GKV_STATIC_SCRATCH_BYTES per GPU that loads the library, held until exit), and
 * it calls no cudaMalloc, cudaFree or any allocating library routine.  Same arguments and result
 * as gkv_mixed_attn_decode otherwise.
 *  - Limit: gkv_decode_workspace_bytes(B, Hq, Hkv, D, nb) must not exceed
 *    GKV_STATIC_SCRATCH_BYTES, else GKV_E_STATIC_SCRATCH is returned and nothing is launched.
 *  - The first call on each device looks up the array's device address (one host-side runtime
 *    query, no allocation); make that first call outside any stream capture.
 *  - All calls on a device share the one array, which keeps the previous call's contents (the
 *    part that must start at zero is cleared on the stream at each call).  Two calls whose
 *    kernels can overlap on the GPU — different streams without an ordering between them —
 *    race on it; serialise them.
 */
#define GKV_STATIC_SCRATCH_BYTES (8u << 20)
int gkv_mixed_attn_decode_static(const float *q, const uint8_t *data, const int64_t *offs,
                                 const void *klo, const void *kstep, const void *vlo, const void *vstep,
                                 const int32_t *level, const int32_t *valid, float *out,
                                 int B, int Hq, int Hkv, int D, int nb, int block, int group,
                                 int64_t stride_bh, int meta_rows, void *stream);

/* LSE merge of `parts` records per output row (mixed_attn.cu:171-200):
 * partials (parts, rows, D+2) fp32 -> out (rows, D) fp32, rows = B*Hq.       */
int gkv_combine_partials(const float *partials, float *out, int parts, int rows, int D, void *stream);

/* ---- packing ---------------------------------------------------------------------
 * Replaces, for whole batches of blocks on the device, quantize_codes
 * (tests/test_cuda_kernel.py:18-33) + pack_bits (geodesia_kv/packed.py:23-40) +
 * build_layout (geodesia_kv/pack_layout.py:14-54).
 *
 *   k, v     (rows, nb, P, D) dense, src_dtype 0 = fp32, 1 = bf16, 2 = fp16
 *   level    target rung per block; offs destination byte offset in the row;
 *            valid real tokens (rows >= valid repeat the last real row, as
 *            blockify does, geodesia_kv/policies.py:126-133)
 *   only blocks b in [b_lo, b_hi) are written.
 * Scale planes are written for rungs 8/4/2 and zeroed for rungs 16 and 1.
 */
int gkv_pack_blocks(const void *k, const void *v, int src_dtype, uint8_t *data, const int64_t *offs,
                    void *klo, void *kstep, void *vlo, void *vstep, const int32_t *level,
                    const int32_t *valid, int rows, int nb, int b_lo, int b_hi, int D, int block,
                    int group, int64_t stride_bh, int meta_rows, void *stream);

/* Demotion without a dense copy: block b of a row is read at rung level_old[b]
 * from offs_old[b], re-quantised from its CURRENT reconstruction to level_new[b]
 * (the batched demotion of geodesia_kv/policies.py:869-908) and written at
 * offs_new[b]; blocks with level_new == level_old are skipped.  Source and
 * destination may be the same bytes (a block is fully read before it is
 * written); distinct blocks must not overlap each other's destination.
 * data_new may equal data_old.                                                 */
int gkv_demote_blocks(const uint8_t *data_old, const int64_t *offs_old, const int32_t *level_old,
                      uint8_t *data_new, const int64_t *offs_new, const int32_t *level_new,
                      void *klo, void *kstep, void *vlo, void *vstep, int rows, int nb, int D,
                      int block, int group, int64_t stride_old, int64_t stride_new, int meta_rows,
                      void *stream);

/* Exact inverse used by tests and the host mirror of PackedBlocks.dequantize:
 * block bytes -> fp32 (rows, nb, P, D) K and V (mixed_attn.cu:93-159).          */
int gkv_unpack_blocks(const uint8_t *data, const int64_t *offs, const void *klo, const void *kstep,
                      const void *vlo, const void *vstep, const int32_t *level, float *k_out,
                      float *v_out, int rows, int nb, int D, int block, int group, int64_t stride_bh,
                      int meta_rows, void *stream);

/* ---- allocator ----------------------------------------------------------------------
 * Replaces the Lagrangian rung allocation of Policy.attend,
 * geodesia_kv/policies.py:810-868, for `problems` independent cache rows.
 *
 *   mass (problems, nb) fp32;  E (problems, nb, 5) fp32 distortion per rung in
 *   ladder order (16, 8, 4, 2, centroid);  idx (problems, nb) int32 current
 *   ladder index;  hot (problems, nb) uint8;  bits[5] HOST floats: resident bits
 *   per rung (policies.py:1582-1596);  target_bits (problems) fp64: budget *
 *   2*nb*P*D;  ratio (problems, nb, 4) fp32 scratch that also returns the
 *   marginal-cost table;  tgt_idx (problems, nb) int32 out.
 * Bit-exact with the reference given the same inputs when mass_power == 1.
 */
int gkv_allocate(const float *mass, const float *E, const int32_t *idx, const uint8_t *hot,
                 const float *bits_host, const double *target_bits, float mass_power, float *ratio,
                 int32_t *tgt_idx, int problems, int nb, void *stream);

/* Distortion table of policies.py:774-808 computed from rung-16 (bf16) blocks
 * of the packed cache: E (rows, nb, 5).  Blocks at other rungs get a zero row
 * (their steps are never taken, see gkv_allocate).                              */
int gkv_block_distortion(const uint8_t *data, const int64_t *offs, const int32_t *level, float *E,
                         int rows, int nb, int D, int block, int group, float value_weight,
                         int64_t stride_bh, int meta_rows, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GEODESIA_KV_B200_H */
