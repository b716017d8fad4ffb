/*
 * geodesia_kv_b200 — C ABI of the B200 (sm_100a) packed-KV decode path.
 *
 * Plain pointers and sizes only; every pointer is a DEVICE pointer unless its
 * comment says "host".  Every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*), never synchronises (gkv_decode_status excepted), allocates
 * no device memory (the caller passes the workspace) and returns 0 or a negative
 * GKV_E_* code; launch errors are returned as GKV_E_CUDA and the CUDA error
 * stays readable through gkv_last_cuda_error().
 *
 * Process-wide state, all of it small: the last CUDA error code; the kernel
 * choice of gkv_set_decode_kernel; per-device caches filled on the first call on
 * a device (multiprocessor count, "large shared memory opted in" flags, the
 * device address of the built-in scratch of gkv_mixed_attn_decode_static); and
 * that scratch array itself.  The caches are written without locks: every
 * writer stores the same value, so concurrent first calls are harmless, but a
 * host that wants no such race makes its first call per device from one thread.
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
 * what selects the tensor-core kernel.  `planned` != 0: the caller passes prebuilt block lists
 * (gkv_mixed_attn_decode_planned), which saves one kernel.  No counterpart in the reference.   */
int gkv_decode_kernel_launches(int B, int Hq, int Hkv, int D, int nb, int group);
int gkv_decode_launch_count(int B, int Hq, int Hkv, int D, int nb, int group, int planned);

/* Kernel choice for every later decode call of the process: 0 = by shape (tensor-core kernel
 * for D in {64,128}, g in {16,32,64}, GQA width <= 8; the CUDA-core kernel otherwise), 1 = always
 * the CUDA-core kernel (exact fp32 arithmetic; used to cross-check the two).  No counterpart in
 * the reference, which has a single kernel.                                                    */
int gkv_set_decode_kernel(int which);

/* Blocks per work item of the tensor-core kernel for every later decode call of the process:
 * 0 = chosen from the problem size (about six items per multiprocessor, between 6 and 64 blocks),
 * 1..64 = fixed.  A tuning and test knob: results do not depend on it, only the split does (and with
 * it gkv_decode_workspace_bytes: query the size after setting the knob).  No counterpart in the
 * reference, whose split is fixed by its launcher (geodesia_kv_cuda/mixed_attn.cu:222-224).      */
int gkv_set_decode_item_blocks(int blocks);


/* What happens when a wait inside the tensor-core kernel runs out.  Every wait of that kernel (on
 * a shared-memory barrier that a copy or another warp completes) gives up after about one second
 * of wall time; the kernel then records a non-zero code in the workspace, all its warps leave,
 * and the merge fills the WHOLE output with NaN — the call itself has long returned GKV_OK, being
 * asynchronous.  gkv_decode_status reads that code back: it copies the status word of the most
 * recent call that used `workspace` to *status_host (0 = completed normally) and SYNCHRONISES
 * `stream` to do so.  A host that never sees NaN outputs need not call it.  The limit is wall
 * time, so a context that is time-sliced or preempted for longer than the limit can trip it.
 * The reference has no such path: its kernel has no waits.                                     */
int gkv_decode_status(const void *workspace, int *status_host, void *stream);

int gkv_mixed_attn_decode(const float *q, const uint8_t *data, const int64_t *offs,
                          const void *klo, const void *kstep, const void *vlo, const void *vstep,
                          const int32_t *level, const int32_t *valid, float *out,
                          void *workspace, size_t workspace_bytes,
                          int B, int Hq, int Hkv, int D, int nb, int block, int group,
                          int64_t stride_bh, int meta_rows, void *stream);

/* The tensor-core kernel walks every cache row's blocks sorted by rung.  Those lists depend only
 * on offs / level / valid, so a caller whose metadata is unchanged since the last call can build
 * them once (gkv_decode_build_plan into gkv_decode_plan_bytes(meta_rows, nb) bytes, 16-byte
 * aligned) and pass them to gkv_mixed_attn_decode_planned, which then launches one kernel less.
 * `plan` may be NULL (the lists are then rebuilt inside the workspace, exactly as
 * gkv_mixed_attn_decode does); `partial` != 0 gives gkv_mixed_attn_decode_partial's output.
 * A stale plan (metadata changed since it was built) gives wrong results, not an error.
 * Extends mixed_attn_decode (geodesia_kv_cuda/mixed_attn.cu:202-244), which re-derives its split
 * on every call.                                                                                */
size_t gkv_decode_plan_bytes(int meta_rows, int nb);
int gkv_decode_build_plan(const int64_t *offs, const int32_t *level, const int32_t *valid, void *plan,
                          int meta_rows, int nb, void *stream);
int gkv_mixed_attn_decode_planned(const float *q, const uint8_t *data, const int64_t *offs,
                                  const void *klo, const void *kstep, const void *vlo, const void *vstep,
                                  const int32_t *level, const int32_t *valid, float *out,
                                  const void *plan, int partial, void *workspace, size_t workspace_bytes,
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

/* Decode attention that also reports where the softmax mass went: mass (B, Hkv, nb) fp32, the mean
 * over a cache row's query heads of the summed softmax weight of each block's tokens — what the
 * reference's allocator is fed with, and what its hook obtains from a second, dense softmax over
 * the keys (geodesia_kv/policies.py:1497-1509; prefill: :1421-1451).  Here it is a by-product of
 * the decode kernel: per block half and head the kernel notes the reference it was using and the
 * sum of its weights, and a small kernel turns those into masses once the heads' final (m, l) are
 * known.  Needs gkv_decode_mass_workspace_bytes() of workspace and a shape the tensor-core kernel
 * takes (D in {64,128}, g in {16,32,64}, GQA width <= 8), else GKV_E_SHAPE.  `plan` as in
 * gkv_mixed_attn_decode_planned (may be NULL).  Blocks with no valid token get mass 0.           */
size_t gkv_decode_mass_workspace_bytes(int B, int Hq, int Hkv, int D, int nb, int group);
int gkv_mixed_attn_decode_mass(const float *q, const uint8_t *data, const int64_t *offs,
                               const void *klo, const void *kstep, const void *vlo, const void *vstep,
                               const int32_t *level, const int32_t *valid, float *out, float *mass,
                               const void *plan, void *workspace, size_t workspace_bytes,
                               int B, int Hq, int Hkv, int D, int nb, int block, int group,
                               int64_t stride_bh, int meta_rows, void *stream);

/* One long sequence split over the GPUs of a node, with the exchange of the per-rank (m, l, o)
 * records done by this library's own merge kernel instead of a collective library: every rank
 * calls this on its slice of the blocks (same q on every rank); the last merge level stores the
 * rank's record of every output row into the INBOX of every rank with plain peer stores, raises
 * the row's sequence number there, waits (bounded, about a second) for the records of all ranks in
 * its own inbox and writes the normalised output — every rank ends up with the full result.
 *
 *   inboxes   HOST array of `world` device pointers: the inbox of every rank as addressable from
 *             this GPU (peer mappings of one symmetric allocation of gkv_exchange_inbox_bytes()
 *             bytes per rank, zero-filled once before the first call)
 *   seq       (B*Hq) ints in LOCAL memory, zero-filled once; counts the calls
 *   xstatus   1 int in local memory, zero-filled once; becomes non-zero when a wait ran out (the
 *             output rows concerned are NaN) and stays so
 * All ranks must make the same sequence of calls with the same inboxes.  A rank that stops calling
 * makes the others' waits run out; it does not hang them.  `plan` as in
 * gkv_mixed_attn_decode_planned (may be NULL).  The reference has no multi-GPU path; this extends
 * its split-and-merge (geodesia_kv_cuda/mixed_attn.cu:58-65, 171-200) across GPUs.               */
size_t gkv_exchange_inbox_bytes(int world, int rows, int D);
/* How long (nanoseconds of wall time) the exchange waits for the other ranks' records before it
 * gives up, for every later call of the process; one second by default.                          */
int gkv_set_exchange_wait_ns(unsigned long long ns);
int gkv_mixed_attn_decode_exchange(const float *q, const uint8_t *data, const int64_t *offs,
                                   const void *klo, const void *kstep, const void *vlo, const void *vstep,
                                   const int32_t *level, const int32_t *valid, float *out, const void *plan,
                                   void *workspace, size_t workspace_bytes, int B, int Hq, int Hkv, int D,
                                   int nb, int block, int group, int64_t stride_bh, int meta_rows,
                                   void *const *inboxes, int rank, int world, int *seq, int *xstatus,
                                   void *stream);

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
 * offs_new[b]; blocks with level_new == level_old are skipped.  A block's
 * destination may overlap its OWN source (a block is fully read before it is
 * written).  Blocks are processed concurrently, so when data_new aliases
 * data_old a block's destination must not overlap any OTHER block's source or
 * destination: demoting in place (offs_new == offs_old) is fine, compacting
 * the row to the left in the same buffer is not — compact into a second buffer. */
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

/* The pack and demote kernels wait, bounded (2 s), for their own bulk copies into shared memory; a
 * wait that runs out makes the kernel set a device-side word and return instead of spinning.  This
 * reads the word of the current device (0 = never happened); it synchronises.                  */
int gkv_maintenance_status(int *status_host);

/* ---- paged pool ----------------------------------------------------------------------
 * The reference's serving plugin keeps one cache object per sequence and frees nothing when a
 * block is demoted (vllm_plugin/kv_cache.py:15-104); its capacity claim (README.md:243-248) needs
 * demotion to give memory back.  The pool form below is what makes that real: every block of
 * every sequence, head and layer is an offset into ONE byte pool, and the four scale planes of a
 * quantised block are stored right behind its bytes, in the order [klo][kstep][vlo][vstep] (fp16,
 * shapes (G, D), (G, D), (64, gv), (64, gv)), so that a block is allocated, moved, shrunk and freed
 * as one piece of gkv_paged_block_bytes(level, D, group) bytes (32768 / 18432 / 10240 / 6144 / 512
 * at D = 128, g = 32).  Slot management (size-class free lists) is the caller's; these entry points
 * only read and write blocks.  Block offsets must be multiples of 16 (of 128 for the tiled copies
 * of the decode kernel to be used; other offsets fall back to a slower copy).  D in {64, 128},
 * group a multiple of 8; else GKV_E_SHAPE.  No counterpart in the reference's C++ (its kernel
 * takes dense side tensors, mixed_attn.cu:202-216).                                          */
size_t gkv_paged_block_bytes(int level, int D, int group);

/* Quantise n blocks from dense rows into pool slots.  Block i reads 64 token rows of D elements
 * starting at element src_off[i] of k and of v (consecutive tokens token_stride elements apart;
 * rows beyond nvalid[i] repeat the last real row; nvalid may be NULL = all 64) and is written at
 * rung level[i] to pool + dst_off[i]; entries with dst_off < 0 are skipped.  ek, ev (n floats,
 * both or neither): += max over the block's tokens of the L2 norm of the quantisation error of
 * K and of V — the radii the reference accumulates when it demotes (policies.py:905-906).    */
int gkv_paged_pack_blocks(const void *k, const void *v, int src_dtype, const int64_t *src_off,
                          int64_t token_stride, const int32_t *nvalid, uint8_t *pool,
                          const int64_t *dst_off, const int32_t *level, float *ek, float *ev, int n,
                          int D, int block, int group, void *stream);

/* Demote n blocks: block i is read at (pool_old + off_old[i], level_old[i]), dequantised exactly
 * and re-quantised at level_new[i] into pool_new + off_new[i] (policies.py:870-908).  Entries
 * with level_new >= level_old or a negative offset are skipped.  pool_new may be pool_old as
 * long as a destination slot overlaps no OTHER entry's source or destination.  ek, ev as above. */
int gkv_paged_demote_blocks(const uint8_t *pool_old, const int64_t *off_old, const int32_t *level_old,
                            uint8_t *pool_new, const int64_t *off_new, const int32_t *level_new,
                            float *ek, float *ev, int n, int D, int block, int group, void *stream);

/* Exact dequantisation of n pool blocks -> fp32 k_out, v_out (n, 64, D) (tests, debugging).   */
int gkv_paged_unpack_blocks(const uint8_t *pool, const int64_t *offs, const int32_t *level,
                            float *k_out, float *v_out, int n, int D, int block, int group,
                            void *stream);

/* Append ONE token to every cache row: k, v (rows, D) of src_dtype are rounded to bf16 and stored
 * as token lens[r] of row r, i.e. into block lens[r] / 64 of the row's table (offs, valid: (rows,
 * cap)), which must already hold a rung-16 slot; valid and lens are advanced on the device.  A row
 * whose next block has no slot (offset < 0, or beyond cap) is left alone and *status is set to 1.
 * What live_cache.py:84-111 of the reference does with torch.cat on dense tensors.            */
int gkv_paged_append_token(const void *k, const void *v, int src_dtype, uint8_t *pool, const int64_t *offs,
                           int32_t *valid, int32_t *lens, int32_t *status, int rows, int cap, int D,
                           int block, void *stream);

/* Decode attention over a block table: offs, level, valid are (B*Hkv, nb) with nb the longest
 * row's block count; shorter rows are padded with valid = 0 entries (never read).  Same output
 * as gkv_mixed_attn_decode on the equivalent row caches (mixed_attn.cu:8-197).  pool_bytes is the
 * size of the pool (the span the copy engine may address).  mass_out may be NULL; otherwise
 * (B*Hkv, nb) fp32 as in gkv_mixed_attn_decode_mass, and the workspace must hold
 * gkv_decode_mass_workspace_bytes().  `plan` as in gkv_mixed_attn_decode_planned (may be NULL). */
int gkv_paged_attn_decode(const float *q, const uint8_t *pool, size_t pool_bytes, const int64_t *offs,
                          const int32_t *level, const int32_t *valid, float *out, float *mass_out,
                          const void *plan, void *workspace, size_t workspace_bytes, int B, int Hq,
                          int Hkv, int D, int nb, int block, int group, void *stream);

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

/* The same for a ragged batch: problem p uses only its first nb_of[p] blocks (arrays keep the
 * common stride nb); blocks beyond that come back with their current index.  nb_of == NULL is
 * gkv_allocate.                                                                              */
int gkv_allocate_ragged(const float *mass, const float *E, const int32_t *idx, const uint8_t *hot,
                        const float *bits_host, const double *target_bits, float mass_power,
                        float *ratio, int32_t *tgt_idx, const int32_t *nb_of, int problems, int nb,
                        void *stream);

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
