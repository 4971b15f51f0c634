/* C ABI of libb200decode.so: hand-written sm_100a kernels for the batch-1 W4A16 LLM decode step.
 *
 * Every entry point takes raw device pointers, plain ints and a CUDA stream (passed as void*; it is a
 * cudaStream_t), launches on that stream without synchronising, allocates nothing and keeps no state, so the
 * whole decode step can be captured into one CUDA graph. The return value is 0 on success or one of the
 * negative B200_ERR_* codes; on an error nothing has been launched. Device pointers marked "16B" must be
 * 16-byte aligned. All activations, weights scales and caches are fp16 unless stated.
 *
 * The first six functions replace, one for one, the raw-pointer launchers that the reference project
 * declares in kernels/bindings.cpp:7-16 and wraps for Python in kernels/bindings.cpp:27-88. The remaining
 * ones are additions (batching, head_dim 128, the bit-exactness probe, step glue).
 */
#ifndef B200DECODE_H_
#define B200DECODE_H_

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_ERR_ARG (-1)    /* null pointer, non-positive size, value out of range */
#define B200_ERR_ALIGN (-2)  /* a pointer that must be 16-byte aligned is not */
#define B200_ERR_SHAPE (-3)  /* a shape this library has no kernel for */
#define B200_ERR_LAUNCH (-4) /* the CUDA runtime refused the launch (see b200_last_cuda_error) */
#define B200_ERR_LIMIT (-5)  /* a size beyond a fixed capacity of the entry point */

/* Library version (major * 100 + minor). */
int b200_version(void);
/* Static text for a B200_ERR_* code. */
const char* b200_strerror(int code);
/* Text of the CUDA error behind the last B200_ERR_LAUNCH on this host thread. */
const char* b200_last_cuda_error(void);

/* y[N] = dequant(W)[N,K] . x[K], fp32 accumulate.
 * Replaces gemv_w4a16_launch (reference kernels/bindings.cpp:7-8, kernels/gemv_w4a16.cu:111-130).
 * Wp: packed int32 [N, K/8] (16B), SZ: half2 (scale, zero) [N, K >> log2G], x: [K] (16B), y: [N].
 * K % 32 == 0, group = 2^log2G >= 32 and divides K.
 * stage 0 = plain one-thread-per-weight kernel. stage >= 1 with R in {1,2,4,8} and warps in 1..8 runs
 * that rows-per-warp / warps-per-block configuration on the CUDA cores; R = 16 runs the segmented CUDA-core kernel;
 * any other R (use 0) lets the library choose: the tensor-core kernel (nibbles as unsigned bytes and x as two signed
 * byte digits per 128-element unit into the integer mma.m16n8k32, exact accumulation, one scale per unit) when
 * K % 128 == 0 and the group size is a multiple of 128, else the segmented one.
 * pf is accepted for signature compatibility and ignored. */
int b200_gemv_w4a16(int stage, int R, int warps, int pf, const void* Wp, const void* SZ, const void* x, void* y,
                    int N, int K, int log2G, void* stream);

/* XOR-reduce `bytes` of device memory with streaming 128-bit loads; the achieved GB/s is the library's own
 * achievable-read-bandwidth figure. sink: 4 writable bytes. unroll: 1, 4 or 8.
 * Replaces bw_read_launch (reference kernels/bindings.cpp:9, kernels/gemv_w4a16.cu:149-153). */
int b200_bw_read(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll, void* stream);

/* Paged split-K decode attention for one sequence, head_dim 64, followed by the combine step.
 * Replaces paged_attention_launch (reference kernels/bindings.cpp:10-12, kernels/paged_attention.cu:429-461).
 * q [n_q, 64]; kc, vc [pages, n_kv, 2^log2P, 64] (16B); bt int32 [pages]; pos int32 [1] on the device, context
 * = pos + 1; PS = tokens per split; scratch o_part fp32 [n_q, max_splits, 64], m_part, l_part fp32
 * [n_q, max_splits]; out [n_q, 64]. n_q / n_kv in {1,2,4,8}. Tokens beyond max_splits * PS are ignored.
 * `version` (1..3, as in the reference, whose three versions are three generations of its kernel) selects the kernel:
 * 1 = K/V by register loads (any page and split size); 2 = K/V pages pulled into a shared-memory ring by bulk async
 * copies, arithmetic on the fp32 pipes; 3 = the same ring with both contractions as warp-level tensor-core MMAs
 * (the fastest; with 8 query heads per KV head the fp32 pipes cannot keep up with HBM). 2 and 3 need pages of 8..64
 * tokens and PS a multiple of the page size and otherwise run as 1. All three meet the same tolerance. */
int b200_paged_attention(int version, const void* q, const void* kc, const void* vc, const int* bt, const int* pos,
                         int n_q, int n_kv, int log2P, int PS, int max_splits, float* o_part, float* m_part,
                         float* l_part, void* out, void* stream);

/* x <- x + delta (fp16 add; delta may be NULL), out <- w * half(float(x) * rsqrt(mean(x^2) + eps)).
 * Replaces add_rmsnorm_launch (reference kernels/bindings.cpp:13, kernels/fused_norm.cu:56-58).
 * x, delta, w, out [H] (16B); H % 8 == 0, H <= 32768. */
int b200_add_rmsnorm(void* x, const void* delta, const void* w, void* out, int H, float eps, void* stream);

/* out[i] = half(silu(gu[i])) * gu[I + i].  gu [2I] (16B), out [I] (16B), I % 8 == 0.
 * Replaces swiglu_launch (reference kernels/bindings.cpp:14, kernels/fused_swiglu.cu:23-26). */
int b200_swiglu(const void* gu, void* out, int I, void* stream);

/* Rotate-half RoPE on q (in place) and k of qkv [(n_q + 2 n_kv) * 64] at position *pos, then store k and v
 * into page bt[pos >> log2P], slot pos & (P - 1) of the caches. cos_t, sin_t fp32 [max_pos, 32].
 * Replaces rope_append_launch (reference kernels/bindings.cpp:15-16, kernels/rope_kv.cu:34-38). */
int b200_rope_append(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt, void* kc,
                     void* vc, int n_q, int n_kv, int log2P, void* stream);

/* ---- additions: no counterpart among the reference's launchers ---- */

/* The same GEMV from a copy of the matrix in "tile layout": per 16-row tile and per 128 columns, the bytes in the
 * order the tensor-core kernel's warps read them (512 B for rows 0-7 of the tile, 512 B for rows 8-15, the 16 rows'
 * (scale, zero)), tiles and column blocks back to back. Every warp load is then one contiguous 512-byte read; on
 * matrices with long rows this is worth 1.5x over the row-major tensors (DRAM locality). b200_gemv_w4a16_tiled_bytes
 * gives the size of the copy (0 if K % 128 != 0), b200_gemv_w4a16_tile_repack fills it once from the quantizer's
 * tensors (group size a multiple of 128), b200_gemv_w4a16_tiled computes y = W x from it (x 8-byte aligned).
 * gate_up != 0 (repack) / swiglu != 0 (GEMV): the matrix is [gate; up] with N = 2 I rows; the copy pairs gate row i
 * with up row i inside a tile, and the GEMV - called with N = I - stores half(silu(gate_i)) * up_i, the result of
 * b200_gemv_w4a16 followed by b200_swiglu, in one launch. */
size_t b200_gemv_w4a16_tiled_bytes(int N, int K, int gate_up);
int b200_gemv_w4a16_tile_repack(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, int gate_up,
                                void* stream);
int b200_gemv_w4a16_tiled(const void* Wt, const void* x, void* y, int N, int K, int swiglu, void* stream);

/* Launch shape of the tensor-core GEMV for one matrix shape, found by measurement instead of the built-in heuristic
 * (the counterpart of the per-shape (stage, R, warps, pf) table the reference grows with scripts/autotune.py:1-58 and
 * reads in runtime/model.py:174-178). layout: 0 row-major tensors (b200_gemv_w4a16 with R = 0), 1 tile layout,
 * 2 paired gate|up tile layout (N = outputs). ksplit in {1, 2, 4, 8} warps share a 16-row tile by splitting K;
 * blocks = thread blocks to launch at most. ksplit = 0 forgets the shape. Host-side table of the process (128 shapes,
 * B200_ERR_LIMIT beyond); set it up before launching from other threads. */
int b200_gemv_w4a16_tune(int layout, int N, int K, int ksplit, int blocks);

/* b200_add_rmsnorm followed by b200_gemv_w4a16_tiled, in one launch: r = x_in + delta (fp16 add; delta may be NULL),
 * x = norm_w * half(float(r) * rsqrt(mean(r^2) + eps)), y = W x (or SwiGLU of it). Every thread block normalises
 * its own copy of the K activations while its first weights are in flight; r goes to x_out, which must not be
 * x_in. All vectors fp16 [K], 8-byte aligned. */
int b200_gemv_w4a16_tiled_norm(const void* Wt, const void* x_in, const void* delta, const void* norm_w, float eps,
                               void* x_out, void* y, int N, int K, int swiglu, void* stream);

/* Like b200_bw_read, but through the path the persistent step kernel uses: each of `blocks` CTAs streams its share
 * of the buffer into a shared-memory ring of `stages` x `stage_bytes` with 1-D bulk async copies. stage_bytes a
 * multiple of 128, stage_bytes * stages <= 226 KB. *sink becomes 0xdead000x if a bounded wait inside gives up. */
int b200_bw_read_bulk(const void* p, size_t bytes, void* sink, int blocks, int stage_bytes, int stages, void* stream);

/* Batched, head_dim-generic form of b200_paged_attention. q [B, n_q, D]; bt int32 [B, bt_stride]; pos int32 [B];
 * o_part [B, n_q, max_splits, D]; m_part, l_part [B, n_q, max_splits]; out [B, n_q, D]. D in {64, 128}.
 * The reference's Python binding hard-wires B = 1 and D = 64 (kernels/bindings.cpp:49-52). */
int b200_paged_attention_batched(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                 const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                                 float* o_part, float* m_part, float* l_part, void* out, void* stream);

/* b200_paged_attention_batched with the kernel chosen by `version` (0 = the library's choice, which is what
 * b200_paged_attention_batched runs; 1..3 as for b200_paged_attention). */
int b200_paged_attention_batched_v(int version, const void* q, const void* kc, const void* vc, const int* bt,
                                   int bt_stride, const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS,
                                   int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                   void* stream);

/* b200_rope_append followed by b200_paged_attention for one sequence, in one partial-kernel launch: qkv is the raw
 * [(n_q + 2 n_kv) * D] vector of the step (left untouched), every block rotates its own query heads, and the block
 * of the last split rotates k, stores k and v at position *pos of the caches and attends to them. The context
 * pos + 1 must lie within max_splits * PS. Pages or splits the ring kernel does not cover run as the two separate
 * kernels. D in {64, 128}; cos_t, sin_t fp32 [max_pos, D/2].
 * arrive: NULL, or n_kv ints that are zero before the first call. With it the split partials are merged inside the
 * same launch by the last block of each kv head to finish (an arrival count, nobody waits; the count is back at zero
 * when the call completes), so no combine kernel is launched: same numbers, one launch less. Calls that share an
 * arrive array must not overlap. */
int b200_rope_paged_attention(void* qkv, const float* cos_t, const float* sin_t, void* kc, void* vc, const int* bt,
                              const int* pos, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                              float* o_part, float* m_part, float* l_part, void* out, int* arrive, void* stream);

/* Health word of the attention kernels on the current device (no counterpart in the reference): *code = 0, or 1 once
 * a thread block gave up a bounded wait for its own asynchronous copies, in which case the outputs of that call are
 * invalid. Every wait inside the library is bounded; this is how a caller learns that one ran out. Synchronises the
 * device. */
int b200_paged_attention_status(int* code);

/* b200_paged_attention for callers that cannot allocate device memory (no counterpart in the reference, whose
 * callers always allocate the partial buffers with torch, runtime/model.py:148-150). The split-K partials go to a
 * fixed array inside the library (about 1 MB per GPU, held until the process exits) instead of caller scratch:
 * n_q <= 64, max_splits <= 32, D in {64, 128}, one sequence; anything larger returns B200_ERR_LIMIT. The first call
 * on a device looks up the array's address (cudaGetSymbolAddress), so make that first call outside any stream
 * capture. All calls on a device share the array: do not let two of them overlap on the GPU. No cudaMalloc, cudaFree
 * or other allocating call is made. q [n_q, D]; kc, vc [pages, n_kv, 2^log2P, D]; out [n_q, D]. */
int b200_paged_attention_noalloc(const void* q, const void* kc, const void* vc, const int* bt, const int* pos, int n_q,
                                 int n_kv, int D, int log2P, int PS, int max_splits, void* out, void* stream);

/* Batched, head_dim-generic form of b200_rope_append. qkv [B, (n_q + 2 n_kv) D]; bt [B, bt_stride]; pos [B];
 * cos_t, sin_t fp32 [max_pos, D/2]. D even, D <= 256. */
int b200_rope_append_batched(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                             int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                             void* stream);

/* Batched forms for the prompt: rows of x / delta / out are H apart, the norm weight is shared; gu [rows, 2I],
 * out [rows, I]. Same arithmetic per row as b200_add_rmsnorm / b200_swiglu. rows <= 65535 for the SwiGLU. */
int b200_add_rmsnorm_batched(void* x, const void* delta, const void* w, void* out, int rows, int H, float eps,
                             void* stream);
int b200_swiglu_batched(const void* gu, void* out, int rows, int I, void* stream);

/* Y[T, N] = X[T, K] . dequant(W)[N, K]^T for the T tokens of a prompt, fp32 accumulation on the tcgen05 tensor cores
 * (accumulator in tensor memory), fp16 out. The reference has no counterpart: it feeds a prompt through its decode
 * step one token at a time (runtime/model.py:267-276) and lists the batched GEMM as cut (RESULTS.md:385-387).
 * Wp int32 [N, K/8] and SZ half2 [N, K >> log2G] are the quantizer's row-major tensors (runtime/quant.py:61-90),
 * X fp16 [T, K] (16B), Y fp16 [T, N]. K % 64 == 0, group = 2^log2G >= 64, T <= b200_gemm_w4a16_max_tokens().
 * The dequantized fp16 weights are those of b200_dequant_w4a16, bit for bit. Waits on the tensor core are bounded:
 * if one runs out the CTA frees its tensor memory and returns, and b200_gemm_w4a16_status reports 1 (sticky). */
int b200_gemm_w4a16(const void* Wp, const void* SZ, const void* X, void* Y, int T, int N, int K, int log2G,
                    void* stream);
int b200_gemm_w4a16_max_tokens(void);
/* Synchronous read of the status word: 0, or 1 once a bounded wait ran out. */
int b200_gemm_w4a16_status(int* code);

/* out fp16 [N, K] (16B) = per-element dequantized weight, bit-identical to the quantizer's dequantize
 * (reference runtime/quant.py:93-97). Used to prove the kernels read the packed format correctly. */
int b200_dequant_w4a16(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, void* stream);

/* x[H] = emb[tok[0], :]; tok is int64 [1] on the device (the reference's step does this with
 * torch.index_select, runtime/model.py:218). emb fp16 [V, H], x 16B; H % 8 == 0. A token outside [0, V) reads row 0
 * instead of memory outside the table. */
int b200_embed_row(const void* emb, const long long* tok, void* x, int H, int V, void* stream);

/* tok[0] = index of the largest fp16 logit (lowest index on ties, NaNs skipped; 0 if every logit is NaN). If pos != NULL: when history
 * != NULL, history[pos[0]] = tok[0] (int64 array long enough for every position); then pos[0] += 1.
 * (torch.argmax and `pos += 1` in the reference's step, runtime/model.py:232-233.) */
int b200_argmax(const void* logits, int V, long long* tok, int* pos, long long* history, void* stream);

/* ---- the whole decode step as one persistent kernel ----
 * Replaces, for one token, the launch sequence of the reference's Model.step() (runtime/model.py:216-233): embedding
 * row, per layer [add+RMSNorm, qkv GEMV, RoPE + KV append, attention, o GEMV, add+RMSNorm, gate|up GEMV, SwiGLU,
 * down GEMV], final norm, LM-head GEMV, argmax into tok, history[pos] = tok, pos += 1. One cooperative launch of
 * `grid` CTAs (one per SM); weights stream through shared-memory rings, CTAs exchange activations through `xchg`.
 * The reference has no such entry point: there the step is ~225 launches issued from Python. */

/* One decoder layer. An array of L of these lives in DEVICE memory. Matrix order in w[]:
 * 0 = [q;k;v] ((n_q + 2 n_kv) D x H), 1 = o (H x n_q D), 2 = [gate;up] (2I x H), 3 = down (H x I). */
typedef struct b200_step_layer {
  const void* w[4];  /* the matrix in tile layout (b200_gemv_w4a16_tile_repack); w[2] with gate_up = 1 */
  const void* sz[4]; /* unused (the tile layout carries scale/zero); set to NULL */
  const void* ln1;   /* fp16 [H] */
  const void* ln2;   /* fp16 [H] */
  void* kc;          /* fp16 [pages, n_kv, P, D] */
  void* vc;
} b200_step_layer;

/* Host-side description of a step; every pointer inside points to device memory. */
typedef struct b200_step_desc {
  const b200_step_layer* layers;
  int L, H, I, n_q, n_kv, D, V, log2G, log2P;
  float eps;
  const void* emb;     /* fp16 [vocab, H] */
  const void* norm_f;  /* fp16 [H] */
  const void* w_head;  /* LM head [V, H] in tile layout (b200_gemv_w4a16_tile_repack, gate_up = 0) */
  const void* sz_head; /* unused; NULL */
  const float* cos_t;  /* fp32 [max_pos, D/2] */
  const float* sin_t;
  const int* bt;       /* int32 block table of the sequence */
  long long* tok;      /* int64 [1]: token to consume; receives the argmax */
  int* pos;            /* int32 [1]: position of tok; incremented */
  long long* history;  /* int64 [max positions] or NULL */
  void* logits;        /* fp16 [V] */
  void* xchg;          /* b200_decode_step_xchg_bytes() bytes, zeroed once by the caller, then owned by the step */
  void* ctrl;          /* 16 bytes, zeroed once: {uint32 completed steps, int32 error, int32 abort, pad} */
  int ctx_cap;         /* largest context (pos + 1) this launch may see */
  int grid;            /* CTAs = SMs of the device */
  long long* trace;    /* NULL. (A library built with -DB200_STEP_TRACE, which the normal build never is, fills an
                        * int64 [grid, 8 + 25 (L + 1)] array here with per-CTA globaltimer values inside every phase.) */
} b200_step_desc;

/* Bytes of exchange memory a step of these dimensions needs. */
size_t b200_decode_step_xchg_bytes(int L, int H, int I, int n_q, int n_kv, int D, int grid);

/* Launch one step. B200_ERR_SHAPE if the dimensions do not fit the kernel (H, n_q D and I multiples of 128, group size
 * a multiple of 128, pages of at most 64 tokens, the shared-memory plan; use the per-operator entry points then),
 * B200_ERR_LIMIT if ctx_cap is beyond what the in-kernel attention holds.
 * Waits inside the kernel are bounded: if one gives up, ctrl.error becomes non-zero (1 tag poll, 2 ring full,
 * 3 ring empty) and the step's outputs are invalid; the caller checks it after synchronising. ctrl.error = 4: tok was
 * outside [0, V) - row 0 of the embedding was used instead and the step completed. A logit vector with no comparable
 * entry (all NaN) yields token 0, as an in-range answer like torch.argmax's. */
int b200_decode_step(const b200_step_desc* d, void* stream);

/* ---- tensor-parallel exchange over NVLink peer memory (one process per GPU, all GPUs in one node) ----
 * No counterpart in the reference, which is single-GPU; the 70B-shape configuration splits o_proj / down_proj by
 * rows and the LM head by vocabulary, and these entry points are the collectives of that split, fused with the
 * operator that follows them. They are the only entry points that own device memory.
 *
 * An exchange block is b200_comm_header_bytes() of flags followed by data slots at caller-chosen offsets (multiples
 * of 16). Every rank allocates one block of the same size (b200_comm_alloc, zero-filled), exports it as a 64-byte
 * CUDA IPC handle (b200_comm_export), sends the handle to its peers by any host channel, and maps theirs
 * (b200_comm_import). `peers` below is a HOST array of W device pointers, peers[r] = rank r's block as this process
 * sees it (peers[rank] = the local block). All ranks must issue the same sequence of exchange calls. */
int b200_comm_header_bytes(void);
int b200_comm_alloc(size_t bytes, void** ptr);
int b200_comm_free(void* ptr);
int b200_comm_export(void* ptr, void* handle64);
int b200_comm_import(const void* handle64, void** ptr);
int b200_comm_unimport(void* ptr);
/* Zero the block's header (flags, step counter, error word). Call on every rank, between two host-side barriers. */
int b200_comm_reset(void* base);
/* How many polls an exchange kernel of this rank spends on one peer before it gives up (0 = the default, about four
 * seconds). A rank that knows its peers answer within microseconds can set a bound of milliseconds, so that a peer
 * that has died is reported quickly. Kept across b200_comm_reset. Synchronises. */
int b200_comm_set_wait_limit(void* base, unsigned int polls);
/* *code = 0, or 1 once a bounded wait for a peer ran out (that call's outputs are untouched and invalid). Synchronises. */
int b200_comm_error(const void* base, int* code);

/* Replaces "NCCL all-reduce, then add_rmsnorm" after a row-split projection. Every rank's GEMV has written its
 * partial fp16 [H] at slot_off of its own block; this sums the W partials (fp32, rank order, rounded to fp16 - the
 * same bits on every rank), then x <- x + sum and out <- RMSNorm(x) * w exactly as b200_add_rmsnorm. One kernel:
 * flag round with the peers (bounded waits), peer loads, norm. H % 8 == 0, H <= 32768. A slot may be reused once
 * another exchange call has completed in between. */
int b200_tp_allreduce_add_rmsnorm(const void* const* peers, int rank, int W, size_t slot_off, void* x, const void* w,
                                  void* out, int H, float eps, void* stream);

/* The row-split projection AND its all-reduce in one kernel (o_proj, down_proj of a tensor-parallel layer): y[N] = sum
 * over the W ranks of (that rank's W_r x_r), every rank calling with its own column shard in tile layout
 * (b200_gemv_w4a16_tile_repack) and its own x. Each thread block pushes the rows it has computed into every rank's
 * exchange region over NVLink as 32-bit words (tag << 16 | fp16 row), tag = the region's call number; after its last
 * row it collects the same rows from its OWN region, where the peers' copies arrive, polling each word until it
 * carries the tag (bounded; on a timeout b200_comm_error = 1 and those rows of y are left alone), and adds the W
 * copies in rank order (fp32, one rounding): bit-identical sums on all ranks, no flag round, no exchange kernel, no
 * NCCL call. All ranks must call with the same N and K (they launch the same grid). y is local memory (fp16 [N],
 * 16-byte aligned); feed it as `delta` to b200_gemv_w4a16_tiled_norm. slot_off: offset, a multiple of 256, of a
 * region of b200_tp_gemv_slot_bytes(N, W) bytes inside every rank's block, used by this call sequence only;
 * successive calls must alternate between at least two such regions (o_proj / down_proj do). N % 8 == 0.
 * B200_ERR_LIMIT if the launch would have more than 1024 thread blocks. W = 1 is allowed (no peer, y = W x). */
size_t b200_tp_gemv_slot_bytes(int N, int W);
int b200_gemv_w4a16_tiled_allreduce(const void* Wt, const void* x, void* y, int N, int K, const void* const* peers,
                                    int rank, int W, size_t slot_off, void* stream);

/* The same exchange with the sum on the consumer's side and no flag round. b200_gemv_w4a16_tiled_push computes this
 * rank's partial rows and pushes them, as 32-bit words (tag << 16 | fp16 row) carrying the slot's call number, into
 * every rank's region; it writes no y and waits for nobody. b200_tp_pushed_add_rmsnorm, launched after it on every
 * rank, polls the W x H words that are (or are about to be) in its OWN region until they carry the call's tag
 * (bounded; on a timeout b200_comm_error = 1 and the outputs are untouched), adds the W copies in rank order (fp32,
 * one rounding: the same bits on every rank), then x <- x + sum, out <- RMSNorm(x) * w as b200_add_rmsnorm, and moves
 * the region's call counter on. A word that carries the tag is its own arrival flag, so the exchange costs one
 * NVLink flight and no system-scope fence. The region is that of b200_tp_gemv_slot_bytes(H, W); the same rules for
 * alternating regions apply. N of the push == H of the consumer. */
int b200_gemv_w4a16_tiled_push(const void* Wt, const void* x, int N, int K, const void* const* peers, int rank, int W,
                               size_t slot_off, void* stream);
int b200_tp_pushed_add_rmsnorm(const void* const* peers, int rank, int W, size_t slot_off, void* x, const void* w,
                               void* out, int H, float eps, void* stream);

/* Replaces the all-gather of the vocabulary-split LM head: dst[r * n + i] = rank r's fp16 shard[i] found at slot_off
 * of its block. Same flag round. dst 16-byte aligned when n % 8 == 0. */
int b200_tp_allgather(const void* const* peers, int rank, int W, size_t slot_off, void* dst, int n, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200DECODE_H_ */
