/*
 * nb200 -- C ABI of the B200 (sm_100a) kernel library behind the HTile translator.
 *
 * Every entry point takes raw device pointers, explicit extents, a dtype code and a CUDA stream
 * (a cudaStream_t passed as void*).  Calls are asynchronous on that stream and never synchronise
 * the device.  Nothing is allocated behind the caller's back: scratch memory is caller-provided
 * and sized by the matching *_workspace_bytes function (the exceptions are nb200_decode_fwd_static, which
 * uses a fixed array built into the library, and nb200_peer_buffer_alloc, whose job is to allocate).  Every function that can fail returns an
 * int: 0 on success, a negative NB200_ERR_* code otherwise, with a thread-local message available
 * from nb200_last_error().  The library is safe to call from one host thread per GPU.
 *
 * Reference interfaces replaced (paths inside the reference project):
 *   - the GPU kernel that src/neptune_mlir/translators/triton.py:63-77 emits for a func.func and
 *     that tests/test_translators.py:184-194 launches as module.<sym_name>[grid](q, k, v, out):
 *     tensors in memref-argument order, output written in place, launch on the current stream.
 *   - tests/golden/flash_attention_triton.py:4-64 is the executable form of the attention program
 *     (tests/data/flash_attention_htile.mlir:11-149) that nb200_attn_fwd implements.
 */
#ifndef NB200_H
#define NB200_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NB200_OK 0
#define NB200_ERR_BAD_ARG (-1)        /* null pointer, non-positive extent, misaligned pointer   */
#define NB200_ERR_UNSUPPORTED (-2)    /* shape / dtype outside what the kernels implement        */
#define NB200_ERR_LAUNCH (-3)         /* the CUDA runtime or driver rejected a call              */
#define NB200_ERR_DEVICE_TIMEOUT (-4) /* a bounded device-side wait expired (see status word)    */
#define NB200_ERR_NCCL (-5)           /* NCCL could not be loaded, or a collective call failed   */

/* dtype codes: element type of the storage tensors */
#define NB200_F16 0
#define NB200_BF16 1
#define NB200_F32 2

/* Number of 32-bit words in a status buffer (see nb200_attn_fwd). */
#define NB200_STATUS_WORDS 4

/* Library version as major*10000 + minor*100 + patch. */
int nb200_version(void);

/* Message of the last failing call on this host thread ("" if none). */
const char *nb200_last_error(void);

/*
 * Fused attention forward: out = softmax(q k^T * scale) v, optionally causal.
 * Replaces the kernel generated from tests/data/flash_attention_htile.mlir:11-149
 * (golden: tests/golden/flash_attention_triton.py:4-64).
 *
 *   q, out : [B, H, Sq, D]   k, v : [B, H, Skv, D]   contiguous, element type `dtype`
 *   scale_log2 : log2(e) * softmax scale (the program's constant at flash_attention_htile.mlir:24);
 *                scores are taken to the exp2 domain exactly as the program does
 *   causal     : query row i sees keys j <= i + (Skv - Sq)
 *   status     : device buffer of NB200_STATUS_WORDS int32, zeroed by the caller, or NULL.  If a
 *                bounded device-side wait expires the kernel records where in status[0..3] and
 *                finishes without completing the output; read it with nb200_status_read.
 *
 * f16 / bf16 with D == 128 (any Sq, Skv) and 16-byte aligned tensors run on tcgen05 tensor cores with
 * TMA-staged tiles (misaligned tensors are NB200_ERR_BAD_ARG, not a fall-back); f32, and f16 / bf16 with another
 * D, run on an exact-fp32 SIMT kernel, which needs D a multiple of 32, D <= 256 and B * H <= 65535 and returns
 * NB200_ERR_UNSUPPORTED otherwise.  The tensor-core path is a persistent kernel whose CTAs take tiles from a
 * counter inside the library: the call enqueues a 4-byte memset of that counter on `stream` in front of the kernel
 * (capturable in a CUDA graph); up to 64 such launches may be in flight on one GPU at a time.
 */
int nb200_attn_fwd(const void *q, const void *k, const void *v, void *out,
                   int B, int H, int Sq, int Skv, int D, int dtype,
                   float scale_log2, int causal, int *status, void *stream);

/* Copies a status buffer to the host after synchronising `stream`; returns NB200_OK if status[0] is clear,
 * NB200_ERR_BAD_ARG if a kernel refused device-side data (code 22: a block-table entry outside the page pool),
 * NB200_ERR_DEVICE_TIMEOUT for every other code (an expired bounded wait). host_out may be NULL.
 * A non-zero status[0] makes later attention and SSD launches that are given the same buffer return at once
 * without touching their outputs, so read it (and zero it) after synchronising whenever a result matters. */
int nb200_status_read(const int *status, int *host_out, void *stream);

/*
 * Split-K flash-decoding with grouped-query attention (no counterpart kernel in the reference; the
 * operator follows the reference's [B, H, S, D] layout convention, flash_attention_htile.mlir:12-15).
 *
 *   q : [B, Hq, D]      k, v : [B, Hkv, Lkv, D]      (f16 or bf16, D == 128, Hq % Hkv == 0)
 *   partials : fp32 [B, Hq, n_splits, D + 2]; per (b, hq, split) the un-normalised output o[D]
 *              followed by m (running maximum, exp2 domain) and l (sum of 2^(x - m))
 *   scale_log2 : log2(e) * softmax scale
 *   status     : device buffer of NB200_STATUS_WORDS int32, zeroed by the caller, or NULL (as for nb200_attn_fwd).
 *                Long splits stream K/V through a ring of bulk copies whose waits are bounded; a wait that
 *                expires records code 21 there and poisons that split's partial with NaN, so the combined
 *                output is NaN rather than a wrong number; nb200_status_read then returns
 *                NB200_ERR_DEVICE_TIMEOUT.
 * Split s covers KV rows [floor(s*Lkv/n_splits), floor((s+1)*Lkv/n_splits)); n_splits <= Lkv, otherwise free
 * (choose it so that n_splits * Hkv * B fills the GPU's resident CTA slots, two per SM, a whole number of times;
 * nb200_decode_auto_splits does that).
 */
size_t nb200_decode_workspace_bytes(int B, int Hq, int D, int n_splits);

int nb200_decode_splitk(const void *q, const void *k, const void *v, float *partials,
                        int B, int Hq, int Hkv, int Lkv, int D, int n_splits, int dtype,
                        float scale_log2, int *status, void *stream);

/*
 * Number of splits that fills the current device's resident CTA slots (two per SM) a whole number of times
 * for a decode of B sequences with Hkv kv heads of Lkv rows: the smallest count of whole waves whose splits
 * are at least 256 rows long, at most max_splits (0 = no limit).  Returns 0 on a bad argument or if the device
 * cannot be queried.  A program whose split count is 0 asks for this choice.
 */
int nb200_decode_auto_splits(int B, int Hkv, int Lkv, int max_splits);

/*
 * Log-sum-exp combine of partials.  Partial (row, split) starts at
 * partials + row * row_stride + split * split_stride (strides in floats), so the same call merges
 * the splits of one GPU (row_stride = n_splits*(D+2), split_stride = D+2) and the per-GPU partials
 * gathered from several GPUs (row_stride = D+2, split_stride = rows*(D+2)).
 *   out_dtype NB200_F16 / NB200_BF16 : out is [rows, D], normalised and rounded
 *   out_dtype NB200_F32              : out is [rows, D + 2] fp32, again a partial (o, m, l),
 *                                      ready to be merged once more
 * partials must be 8-byte aligned with even strides; out 8-byte aligned for 16-bit outputs (it is written four
 * elements at a time), 4-byte aligned for fp32.
 */
int nb200_decode_combine(const float *partials, void *out, int rows, int D, int n_splits,
                         long long row_stride, long long split_stride, int out_dtype, void *stream);

/*
 * Split-K decode over a paged KV cache with per-sequence lengths (no counterpart in the reference): the
 * serving-side form of nb200_decode_splitk.  A page holds 64 consecutive rows of one sequence for every kv head.
 *
 *   q            : [B, Hq, D]
 *   k_pages, v_pages : [num_pages, Hkv, page_size, D] page pools (f16 or bf16, D == 128, page_size == 64)
 *   block_table  : int32 [B, max_pages]; entry p of row b is the pool index of page p of sequence b
 *                  (entries at and beyond ceil(seq_lens[b] / page_size) are not read)
 *   seq_lens     : int32 [B], rows of each sequence; 0 is allowed and yields a zero output row; a length
 *                  beyond max_pages * page_size is cut to that (the table row addresses no more)
 *   num_pages    : pages in each pool.  The table lives on the device, so the host cannot check it: the kernel
 *                  does.  An entry outside [0, num_pages) is never dereferenced; the split that met it gets a
 *                  NaN partial and `status` (as for nb200_decode_splitk, may be NULL) records code 22 with the
 *                  offending entry, which nb200_status_read reports as NB200_ERR_BAD_ARG.
 *   partials     : fp32 [B, Hq, n_splits, D + 2] as for nb200_decode_splitk; merge with nb200_decode_combine
 * Split s of sequence b covers pages [floor(s*np/n_splits), floor((s+1)*np/n_splits)) with np its page count.
 * Every page reaches shared memory as one TMA bulk copy per operand.
 */
int nb200_decode_paged_splitk(const void *q, const void *k_pages, const void *v_pages, const int *block_table,
                              const int *seq_lens, float *partials, int B, int Hq, int Hkv, int num_pages,
                              int max_pages, int page_size, int D, int n_splits, int dtype, float scale_log2,
                              int *status, void *stream);

/*
 * Merge of a single-sequence decode whose KV cache is split along its length over the ranks of an
 * NCCL communicator (no counterpart in the reference).  Each rank first runs nb200_decode_splitk on
 * its slice and nb200_decode_combine with out_dtype NB200_F32, which leaves one partial per query
 * head; this call all-gathers them and combines across ranks, so every rank ends with the output.
 *
 *   local_partial : fp32 [rows, D + 2], this rank's partials (rows = B * Hq)
 *   gathered      : fp32 [world, rows, D + 2] scratch (nb200_decode_merge_workspace_bytes)
 *   out           : [rows, D] in out_dtype (or [rows, D + 2] fp32 for NB200_F32)
 *   nccl_comm     : the caller's ncclComm_t, whose size must equal `world`
 * NCCL is resolved at run time from the library the process has loaded (else $NEPTUNE_B200_NCCL, else
 * libnccl.so.2); the collective and the combine kernel are enqueued on `stream`.  Like every NCCL
 * collective, all ranks of the communicator must make the call.
 */
size_t nb200_decode_merge_workspace_bytes(int rows, int D, int world);
int nb200_decode_merge_nccl(const float *local_partial, float *gathered, void *out, int rows, int D,
                            int world, int out_dtype, void *nccl_comm, void *stream);

/*
 * The same merge as ONE kernel over peer-mapped memory, without a library collective (no counterpart in the
 * reference).  Every rank owns a symmetric buffer of nb200_decode_merge_peer_workspace_bytes(...) bytes, zeroed
 * once and mapped into every other rank's address space; `peer_buffers` is a HOST array of `world` device
 * pointers, entry r being rank r's buffer as this process sees it (entry `rank` is the rank's own).  The kernel
 * stores this rank's partial into every rank's buffer with plain stores over NVLink, releases one flag per
 * destination, waits until the partials of all ranks have arrived in its own buffer, and combines.  No multicast
 * is used anywhere.
 *
 *   generation : the call's sequence number, the same on every rank, starting at 1 and growing by one per call
 *                (the two halves of the buffer alternate with it, so calls need no clearing in between)
 *   wait_ns    : limit of the wait for the other ranks' partials.  If it expires, `out` is left untouched and
 *                status (NB200_STATUS_WORDS int32, zeroed by the caller, may be NULL) records code 31, the rank
 *                that never arrived and the generation; nb200_status_read then returns NB200_ERR_DEVICE_TIMEOUT.
 * All ranks must make the call, each on its own GPU; the kernels meet through the flags.
 */
size_t nb200_decode_merge_peer_workspace_bytes(int rows, int D, int world);
int nb200_decode_merge_peer(const float *local_partial, void *const *peer_buffers, void *out, int rows, int D,
                            int world, int rank, unsigned generation, int out_dtype, long long wait_ns,
                            int *status, void *stream);

/*
 * The whole sharded single-sequence decode of one rank as ONE kernel launch: split-K over this rank's slice of
 * the cache, the combine of its splits, the push of the rank's partial into every peer's buffer, the bounded
 * wait for the others and the final merge -- the stages handed over by "the last CTA to finish does the next
 * one" tickets, so no CTA waits for another CTA of the launch (no counterpart in the reference).
 *
 *   q : [1, Hq, D]   k, v : [1, Hkv, Lkv, D], this rank's slice   out : [Hq, D] in out_dtype ([Hq, D + 2] fp32 for NB200_F32)
 *   workspace    : nb200_decode_sharded_workspace_bytes(...) bytes, 256-byte aligned, ZEROED ONCE by the caller
 *                  before the first call (ticket counters that the kernel resets itself, the rank's partial, the
 *                  per-split partials)
 *   peer_buffers, generation, wait_ns, status : as for nb200_decode_merge_peer (buffers sized with rows = Hq);
 *                  with world == 1 they are not used and the call is a one-launch decode of one sequence
 * n_splits * Hkv CTAs are launched; choose n_splits so that they fill the GPU's resident slots (two per SM) once.
 * The rows of a kv head are not cut into n_splits fixed ranges: its CTAs take chunks of 128 rows from a counter in
 * the workspace, so CTAs that get a smaller share of their SM do fewer chunks and all end together.
 */
size_t nb200_decode_sharded_workspace_bytes(int Hq, int Hkv, int D, int n_splits);
int nb200_decode_sharded_fwd(const void *q, const void *k, const void *v, void *workspace, void *const *peer_buffers,
                             void *out, int Hq, int Hkv, int Lkv, int D, int n_splits, int dtype, float scale_log2,
                             int world, int rank, unsigned generation, int out_dtype, long long wait_ns, int *status,
                             void *stream);

/*
 * Allocation and CUDA-IPC mapping of such a symmetric buffer: the only entry points of the library that
 * allocate device memory, and they say so by name (a host with its own way of mapping peer memory does not
 * need them).  alloc: cudaMalloc + clear + export a 64-byte handle; open: map another process's buffer from
 * its handle (peer access is enabled on first use); close / free: undo them.  Synchronous; set-up time only.
 */
int nb200_peer_buffer_alloc(size_t bytes, void **ptr, unsigned char *handle64);
int nb200_peer_buffer_open(const unsigned char *handle64, void **ptr);
int nb200_peer_buffer_close(void *ptr);
int nb200_peer_buffer_free(void *ptr);

/*
 * Split-K decode plus combine for callers that may not allocate (no counterpart in the reference).
 *
 * Who needs it: a decode step issued from a serving loop whose memory plan was fixed at start-up.
 * Such a host has handed whatever HBM was left to its KV cache, so a cudaMalloc for the partials can
 * simply fail, and it must not call cudaMalloc / cudaFree in steady state anyway because both
 * synchronise the whole device and stall every other stream of the server; a plugin embedded in a
 * framework that owns the device allocator is in the same position.  This entry point therefore
 * takes only inputs and the output: the per-split partials go to a fixed scratch array compiled
 * into the library (NB200_DECODE_STATIC_SCRATCH_BYTES, resident on every GPU that loads the library
 * until the process exits).  It calls no cudaMalloc, cudaFree or any other allocating routine.
 *
 *   arguments as nb200_decode_splitk, with `out` [B, Hq, D] in `dtype` as nb200_decode_combine writes it
 *   limit: B * Hq * n_splits * (D + 2) * 4 bytes <= NB200_DECODE_STATIC_SCRATCH_BYTES, otherwise
 *          NB200_ERR_UNSUPPORTED with a message naming both sizes (use the workspace entry points then)
 *
 * The first call on a device looks up the scratch array's device address (cudaGetSymbolAddress,
 * once per device, with that device current); make that first call during start-up, before any
 * stream capture begins.  All calls on a device share the one array, which keeps whatever the last
 * call left in it; nothing needs clearing because every slot that is read is written first, but two
 * calls whose kernels can overlap on the GPU (different streams, no dependency) race on it.
 */
#define NB200_DECODE_STATIC_SCRATCH_BYTES (4u << 20)

int nb200_decode_fwd_static(const void *q, const void *k, const void *v, void *out,
                            int B, int Hq, int Hkv, int Lkv, int D, int n_splits, int dtype,
                            float scale_log2, void *stream);

/*
 * Mamba-1 selective scan forward (no counterpart in the reference).
 *   u, delta, z, out : [B, Dm, L] (L contiguous), f16 or bf16; delta already soft-plused
 *   A : fp32 [Dm, N]   Bm, Cm : [B, N, L]   Dskip : fp32 [Dm]   N == 16
 *   h <- exp(delta*A) h + delta*Bm*u ;  y = sum_n Cm h + Dskip u ;  out = y * silu(z)
 * L must be a multiple of 64 and Dm a multiple of 32.
 */
int nb200_selective_scan_fwd(const void *u, const void *delta, const float *A, const void *Bm,
                             const void *Cm, const float *Dskip, const void *z, void *out,
                             int B, int Dm, int L, int N, int dtype, void *stream);

/*
 * Mamba-2 SSD chunked scan forward (no counterpart in the reference).
 *   x, y : [B, L, H, P]   dt : fp32 [B, L, H] (already soft-plused)   A : fp32 [H]
 *   Bm, Cm : [B, L, G, N]  (head h reads group h / (H / G))
 *   workspace : nb200_ssd_workspace_bytes(...) bytes of device memory, 16-byte aligned.  It starts with a status
 *               buffer (NB200_STATUS_WORDS int32) that the call clears and in which an expired device-side wait
 *               is recorded; read it with nb200_status_read.  The recurrent state itself stays on chip.  The
 *               rest is used only when the call cuts the sequences into segments so that a problem with few
 *               (batch, head) pairs still fills the GPU: the fp32 state entering each later segment is prepared
 *               there by one more kernel before the main one (two launches instead of one;
 *               nb200_ssd_launches tells which).  The size does not depend on the device.
 * P == 64, N == 128, chunk in {64, 128, 256}, L a multiple of 128 and of chunk.  The kernel walks the
 * sequence in steps of 128 rows whatever `chunk` says; the result does not depend on the chunk length
 * beyond rounding.  A CTA evaluates two heads that share B and C (H / G even), otherwise one.
 */
size_t nb200_ssd_workspace_bytes(int B, int L, int H, int P, int N, int G, int chunk);

/* Kernel launches that nb200_ssd_chunk_scan_fwd makes for this problem on the current device: 1, or 2 when the
 * sequences are cut into segments.  0 for an unsupported shape. */
int nb200_ssd_launches(int B, int L, int H, int P, int N, int G, int chunk);

int nb200_ssd_chunk_scan_fwd(const void *x, const float *dt, const float *A, const void *Bm,
                             const void *Cm, void *y, void *workspace,
                             int B, int L, int H, int P, int N, int G, int chunk, int dtype,
                             void *stream);

#ifdef __cplusplus
}
#endif

#endif /* NB200_H */
