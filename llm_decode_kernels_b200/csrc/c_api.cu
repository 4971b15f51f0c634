// extern "C" boundary of libb200decode.so: argument checks, then one dispatch per call. Declarations and the
// per-function contract are in include/b200decode.h. Checks mirror the ones the reference performs in its
// Python binding before launching (kernels/bindings.cpp:18-24, 29-35, 47-56, 66-69, 76-77, 84-85), so a bad call
// fails on the host with a code instead of faulting on the device.
#include "../../include/b200decode.h"
#include "common.cuh"
#include "decode_step.h"
#include <string.h>

namespace b200 {
cudaError_t gemv_w4a16_dispatch(int stage, int R, int warps, const void* Wp, const void* SZ, const void* x, void* y,
                                int N, int K, int log2G, cudaStream_t st);
size_t gemv_tiled_bytes(int N, int K, int gate_up);
bool gemv_mma_tune(int mode, int N, int K, int ksplit, int blocks);
cudaError_t gemv_tile_repack_dispatch(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, int gate_up,
                                      cudaStream_t st);
cudaError_t gemv_w4a16_tiled_dispatch(const void* Wt, const void* x, void* y, int N, int K, int swiglu,
                                      cudaStream_t st);
cudaError_t gemv_w4a16_tiled_norm_dispatch(const void* Wt, const void* x_in, const void* delta, const void* norm_w,
                                           float eps, void* x_out, void* y, int N, int K, int swiglu, cudaStream_t st);
cudaError_t gemv_w4a16_tiled_allreduce_dispatch(const void* Wt, const void* x, void* y, int N, int K,
                                                const void* const* peers, int rank, int W, size_t slot_off,
                                                int tagged, cudaStream_t st);
cudaError_t tp_pushed_add_rmsnorm_dispatch(const void* const* peers, int rank, int W, size_t off, void* x, const void* w,
                                           void* out, int H, float eps, cudaStream_t st);
size_t gemv_allreduce_slot_bytes(int N, int W);
cudaError_t dequant_w4a16_dispatch(const void* Wp, const void* SZ, void* out, int N, int K, int log2G,
                                   cudaStream_t st);
cudaError_t add_rmsnorm_dispatch(void* x, const void* delta, const void* w, void* out, int rows, int H, float eps,
                                 cudaStream_t st);
cudaError_t swiglu_dispatch(const void* gu, void* out, int rows, int I, cudaStream_t st);
cudaError_t prefill_gemm_dispatch(const void* Wp, const void* SZ, const void* X, void* Y, int T, int N, int K, int log2G,
                                  cudaStream_t st);
int prefill_gemm_max_tokens();
cudaError_t prefill_gemm_status(int* code);
cudaError_t rope_append_dispatch(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                                 int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                                 cudaStream_t st);
cudaError_t embed_row_dispatch(const void* emb, const long long* tok, void* x, int H, int V, cudaStream_t st);
cudaError_t argmax_dispatch(const void* logits, int V, long long* tok, int* pos, long long* history,
                            cudaStream_t st);
cudaError_t bw_read_dispatch(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll,
                             cudaStream_t st);
cudaError_t bw_read_bulk_dispatch(const void* p, size_t bytes, void* sink, int blocks, int stage_bytes, int stages,
                                  cudaStream_t st);
cudaError_t paged_attention_status(int* code);
cudaError_t rope_paged_attention_dispatch(void* qkv, const float* cos_t, const float* sin_t, void* kc, void* vc,
                                          const int* bt, const int* pos, int n_q, int n_kv, int D, int log2P, int PS,
                                          int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                          int* arrive, cudaStream_t st);
cudaError_t tp_allreduce_add_rmsnorm_dispatch(const void* const* peers, int rank, int W, size_t off, void* x,
                                              const void* w, void* out, int H, float eps, cudaStream_t st);
cudaError_t tp_allgather_dispatch(const void* const* peers, int rank, int W, size_t off, void* dst, int n,
                                  cudaStream_t st);
int comm_header_bytes();
int comm_max_ranks();
int comm_error_offset();
int comm_limit_offset();
cudaError_t paged_attention_dispatch(int version, const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                     const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS,
                                     int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                     cudaStream_t st);
}  // namespace b200

namespace {
thread_local cudaError_t g_last_cuda = cudaSuccess;

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int finish(cudaError_t e) {
  if (e == cudaSuccess) return B200_OK;
  g_last_cuda = e;
  return B200_ERR_LAUNCH;
}
inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

namespace b200 {
void record_cuda_error(cudaError_t e) { g_last_cuda = e; }
}  // namespace b200

#define REQUIRE(cond, code) \
  do {                      \
    if (!(cond)) return (code); \
  } while (0)

extern "C" {

int b200_version(void) { return 100; }

const char* b200_strerror(int code) {
  switch (code) {
    case B200_OK: return "ok";
    case B200_ERR_ARG: return "bad argument (null pointer, non-positive size or value out of range)";
    case B200_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case B200_ERR_SHAPE: return "unsupported shape";
    case B200_ERR_LAUNCH: return "CUDA launch failed";
    case B200_ERR_LIMIT: return "size exceeds the fixed capacity of this entry point";
    default: return "unknown b200 status";
  }
}

const char* b200_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda); }

int b200_gemv_w4a16(int stage, int R, int warps, int pf, const void* Wp, const void* SZ, const void* x, void* y,
                    int N, int K, int log2G, void* stream) {
  (void)pf;
  REQUIRE(Wp && SZ && x && y && N > 0 && K > 0 && stage >= 0, B200_ERR_ARG);
  REQUIRE(log2G >= 5 && log2G < 31, B200_ERR_SHAPE);
  REQUIRE(K % 32 == 0 && K % (1 << log2G) == 0, B200_ERR_SHAPE);
  REQUIRE(K <= 65536, B200_ERR_SHAPE);  // x is staged in shared memory (2 bytes per element)
  REQUIRE(aligned16(Wp) && aligned16(x), B200_ERR_ALIGN);
  REQUIRE((reinterpret_cast<uintptr_t>(SZ) & 3u) == 0 && (reinterpret_cast<uintptr_t>(y) & 1u) == 0, B200_ERR_ALIGN);
  return finish(b200::gemv_w4a16_dispatch(stage, R, warps, Wp, SZ, x, y, N, K, log2G, S(stream)));
}

size_t b200_gemv_w4a16_tiled_bytes(int N, int K, int gate_up) {
  if (N <= 0 || K <= 0 || K % 128 || (gate_up && N % 2)) return 0;
  return b200::gemv_tiled_bytes(N, K, gate_up);
}

int b200_gemv_w4a16_tile_repack(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, int gate_up,
                                void* stream) {
  REQUIRE(Wp && SZ && out && N > 0 && K > 0, B200_ERR_ARG);
  REQUIRE(K % 128 == 0 && log2G >= 7 && log2G < 31 && K % (1 << log2G) == 0 && !(gate_up && N % 2), B200_ERR_SHAPE);
  REQUIRE(aligned16(Wp) && aligned16(out), B200_ERR_ALIGN);
  return finish(b200::gemv_tile_repack_dispatch(Wp, SZ, out, N, K, log2G, gate_up, S(stream)));
}

int b200_gemv_w4a16_tiled(const void* Wt, const void* x, void* y, int N, int K, int swiglu, void* stream) {
  REQUIRE(Wt && x && y && N > 0 && K > 0, B200_ERR_ARG);
  REQUIRE(K % 128 == 0, B200_ERR_SHAPE);
  REQUIRE(K <= 65536, B200_ERR_LIMIT);
  REQUIRE(aligned16(Wt) && (reinterpret_cast<uintptr_t>(x) & 7u) == 0, B200_ERR_ALIGN);
  return finish(b200::gemv_w4a16_tiled_dispatch(Wt, x, y, N, K, swiglu, S(stream)));
}

int b200_gemv_w4a16_tiled_norm(const void* Wt, const void* x_in, const void* delta, const void* norm_w, float eps,
                               void* x_out, void* y, int N, int K, int swiglu, void* stream) {
  REQUIRE(Wt && x_in && norm_w && x_out && y && N > 0 && K > 0 && x_out != x_in, B200_ERR_ARG);
  REQUIRE(K % 128 == 0, B200_ERR_SHAPE);
  REQUIRE(K <= 65536, B200_ERR_LIMIT);
  auto aligned8 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7u) == 0; };
  REQUIRE(aligned16(Wt) && aligned8(x_in) && aligned8(norm_w) && aligned8(x_out) && (!delta || aligned8(delta)),
          B200_ERR_ALIGN);
  return finish(b200::gemv_w4a16_tiled_norm_dispatch(Wt, x_in, delta, norm_w, eps, x_out, y, N, K, swiglu, S(stream)));
}

int b200_gemv_w4a16_tune(int layout, int N, int K, int ksplit, int blocks) {
  REQUIRE(layout >= 0 && layout <= 2 && N > 0 && K > 0 && K % 128 == 0, B200_ERR_ARG);
  REQUIRE(ksplit == 0 || ((ksplit == 1 || ksplit == 2 || ksplit == 4 || ksplit == 8) && blocks > 0), B200_ERR_ARG);
  return b200::gemv_mma_tune(layout, N, K, ksplit, blocks) ? B200_OK : B200_ERR_LIMIT;
}

int b200_bw_read(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll, void* stream) {
  REQUIRE(p && sink && bytes >= 16 && blocks > 0 && threads > 0 && threads <= 1024, B200_ERR_ARG);
  REQUIRE(aligned16(p), B200_ERR_ALIGN);
  return finish(b200::bw_read_dispatch(p, bytes, sink, blocks, threads, unroll, S(stream)));
}

int b200_bw_read_bulk(const void* p, size_t bytes, void* sink, int blocks, int stage_bytes, int stages, void* stream) {
  REQUIRE(p && sink && blocks > 0 && stage_bytes >= 1024 && stages >= 2 && stages <= 32, B200_ERR_ARG);
  REQUIRE(stage_bytes % 128 == 0 && (size_t)stage_bytes * stages + 512 <= 227 * 1024, B200_ERR_SHAPE);
  REQUIRE(bytes >= (size_t)stage_bytes * blocks, B200_ERR_ARG);
  REQUIRE(aligned16(p), B200_ERR_ALIGN);
  return finish(b200::bw_read_bulk_dispatch(p, bytes, sink, blocks, stage_bytes, stages, S(stream)));
}

static int attention_entry(int version, const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                           const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                           float* o_part, float* m_part, float* l_part, void* out, void* stream) {
  REQUIRE(q && kc && vc && bt && pos && out, B200_ERR_ARG);
  REQUIRE(B > 0 && B <= 65535 && n_q > 0 && n_kv > 0 && PS > 0 && max_splits > 0 && max_splits <= 65535 &&
              bt_stride > 0 && log2P >= 0 && log2P < 16 && version >= 0 && version <= 3,
          B200_ERR_ARG);
  REQUIRE(max_splits == 1 || (o_part && m_part && l_part), B200_ERR_ARG);
  REQUIRE(D == 64 || D == 128, B200_ERR_SHAPE);
  REQUIRE(n_q % n_kv == 0, B200_ERR_SHAPE);
  const int hpg = n_q / n_kv;
  REQUIRE(hpg == 1 || hpg == 2 || hpg == 4 || hpg == 8, B200_ERR_SHAPE);
  REQUIRE(aligned16(kc) && aligned16(vc), B200_ERR_ALIGN);
  return finish(b200::paged_attention_dispatch(version, q, kc, vc, bt, bt_stride, pos, B, n_q, n_kv, D, log2P, PS,
                                               max_splits, o_part, m_part, l_part, out, S(stream)));
}

int b200_paged_attention_batched(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                 const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                                 float* o_part, float* m_part, float* l_part, void* out, void* stream) {
  return attention_entry(0, q, kc, vc, bt, bt_stride, pos, B, n_q, n_kv, D, log2P, PS, max_splits, o_part, m_part,
                         l_part, out, stream);
}

int b200_paged_attention_batched_v(int version, const void* q, const void* kc, const void* vc, const int* bt,
                                   int bt_stride, const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS,
                                   int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                   void* stream) {
  return attention_entry(version, q, kc, vc, bt, bt_stride, pos, B, n_q, n_kv, D, log2P, PS, max_splits, o_part,
                         m_part, l_part, out, stream);
}

int b200_paged_attention(int version, const void* q, const void* kc, const void* vc, const int* bt, const int* pos,
                         int n_q, int n_kv, int log2P, int PS, int max_splits, float* o_part, float* m_part,
                         float* l_part, void* out, void* stream) {
  REQUIRE(version >= 1 && version <= 3, B200_ERR_ARG);
  return attention_entry(version, q, kc, vc, bt, 1 << 30, pos, 1, n_q, n_kv, 64, log2P, PS, max_splits, o_part, m_part,
                         l_part, out, stream);
}

int b200_rope_paged_attention(void* qkv, const float* cos_t, const float* sin_t, void* kc, void* vc, const int* bt,
                              const int* pos, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                              float* o_part, float* m_part, float* l_part, void* out, int* arrive, void* stream) {
  REQUIRE(qkv && cos_t && sin_t && kc && vc && bt && pos && out, B200_ERR_ARG);
  REQUIRE(n_q > 0 && n_kv > 0 && PS > 0 && max_splits > 0 && max_splits <= 65535 && log2P >= 0 && log2P < 16,
          B200_ERR_ARG);
  REQUIRE(max_splits == 1 || (o_part && m_part && l_part), B200_ERR_ARG);
  REQUIRE(D == 64 || D == 128, B200_ERR_SHAPE);
  REQUIRE(n_q % n_kv == 0, B200_ERR_SHAPE);
  const int hpg = n_q / n_kv;
  REQUIRE(hpg == 1 || hpg == 2 || hpg == 4 || hpg == 8, B200_ERR_SHAPE);
  REQUIRE(aligned16(kc) && aligned16(vc) && aligned16(qkv) && aligned16(cos_t) && aligned16(sin_t), B200_ERR_ALIGN);
  return finish(b200::rope_paged_attention_dispatch(qkv, cos_t, sin_t, kc, vc, bt, pos, n_q, n_kv, D, log2P, PS,
                                                    max_splits, o_part, m_part, l_part, out, arrive, S(stream)));
}

int b200_paged_attention_status(int* code) {
  REQUIRE(code, B200_ERR_ARG);
  return finish(b200::paged_attention_status(code));
}

int b200_add_rmsnorm_batched(void* x, const void* delta, const void* w, void* out, int rows, int H, float eps,
                             void* stream) {
  REQUIRE(x && w && out && H > 0 && rows > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(H <= 32768, B200_ERR_LIMIT);
  REQUIRE(aligned16(x) && aligned16(w) && aligned16(out) && aligned16(delta), B200_ERR_ALIGN);
  return finish(b200::add_rmsnorm_dispatch(x, delta, w, out, rows, H, eps, S(stream)));
}

int b200_add_rmsnorm(void* x, const void* delta, const void* w, void* out, int H, float eps, void* stream) {
  return b200_add_rmsnorm_batched(x, delta, w, out, 1, H, eps, stream);
}

int b200_swiglu_batched(const void* gu, void* out, int rows, int I, void* stream) {
  REQUIRE(gu && out && I > 0 && rows > 0, B200_ERR_ARG);
  REQUIRE(I % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(rows <= 65535, B200_ERR_LIMIT);
  REQUIRE(aligned16(gu) && aligned16(out), B200_ERR_ALIGN);
  return finish(b200::swiglu_dispatch(gu, out, rows, I, S(stream)));
}

int b200_swiglu(const void* gu, void* out, int I, void* stream) { return b200_swiglu_batched(gu, out, 1, I, stream); }

int b200_gemm_w4a16(const void* Wp, const void* SZ, const void* X, void* Y, int T, int N, int K, int log2G,
                    void* stream) {
  REQUIRE(Wp && SZ && X && Y && T > 0 && N > 0 && K > 0, B200_ERR_ARG);
  REQUIRE(log2G >= 6 && log2G < 31 && K % 64 == 0 && K % (1 << log2G) == 0, B200_ERR_SHAPE);
  REQUIRE(T <= b200::prefill_gemm_max_tokens(), B200_ERR_LIMIT);
  REQUIRE(aligned16(X), B200_ERR_ALIGN);
  return finish(b200::prefill_gemm_dispatch(Wp, SZ, X, Y, T, N, K, log2G, S(stream)));
}

int b200_gemm_w4a16_max_tokens(void) { return b200::prefill_gemm_max_tokens(); }

int b200_gemm_w4a16_status(int* code) {
  REQUIRE(code, B200_ERR_ARG);
  return finish(b200::prefill_gemm_status(code));
}

int b200_rope_append_batched(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                             int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                             void* stream) {
  REQUIRE(qkv && cos_t && sin_t && pos && bt && kc && vc, B200_ERR_ARG);
  REQUIRE(B > 0 && B <= 65535 && n_q > 0 && n_kv > 0 && bt_stride > 0 && log2P >= 0 && log2P < 16, B200_ERR_ARG);
  REQUIRE(D >= 2 && D % 2 == 0 && D <= 256, B200_ERR_SHAPE);
  return finish(b200::rope_append_dispatch(qkv, cos_t, sin_t, pos, bt, bt_stride, kc, vc, B, n_q, n_kv, D, log2P,
                                           S(stream)));
}

int b200_rope_append(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt, void* kc,
                     void* vc, int n_q, int n_kv, int log2P, void* stream) {
  return b200_rope_append_batched(qkv, cos_t, sin_t, pos, bt, 1 << 30, kc, vc, 1, n_q, n_kv, 64, log2P, stream);
}

int b200_dequant_w4a16(const void* Wp, const void* SZ, void* out, int N, int K, int log2G, void* stream) {
  REQUIRE(Wp && SZ && out && N > 0 && K > 0, B200_ERR_ARG);
  REQUIRE(log2G >= 3 && log2G < 31 && K % 8 == 0 && K % (1 << log2G) == 0, B200_ERR_SHAPE);
  REQUIRE(aligned16(out), B200_ERR_ALIGN);
  return finish(b200::dequant_w4a16_dispatch(Wp, SZ, out, N, K, log2G, S(stream)));
}

int b200_embed_row(const void* emb, const long long* tok, void* x, int H, int V, void* stream) {
  REQUIRE(emb && tok && x && H > 0 && V > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(aligned16(emb) && aligned16(x), B200_ERR_ALIGN);
  return finish(b200::embed_row_dispatch(emb, tok, x, H, V, S(stream)));
}

static inline int align_up(int v, int a) { return (v + a - 1) / a * a; }

#ifndef B200_STEP_UPS
#define B200_STEP_UPS 32   // tile-unit blocks per ring stage of the persistent step (build-time knob for measurements)
#endif

size_t b200_decode_step_xchg_bytes(int L, int H, int I, int n_q, int n_kv, int D, int grid) {
  if (grid <= 0 || n_q <= 0) return 0;
  const size_t per_layer = b200::step_words_per_layer(H, I, n_q, n_kv, D, b200::step_att_slices(grid, n_q));
  return (per_layer * L + (size_t)grid * 4) * sizeof(uint32_t);
}

int b200_decode_step(const b200_step_desc* d, void* stream) {
  static_assert(sizeof(b200_step_layer) == sizeof(b200::StepLayer), "layer structs must match");
  REQUIRE(d && d->layers && d->emb && d->norm_f && d->w_head && d->cos_t && d->sin_t && d->bt &&
              d->tok && d->pos && d->logits && d->xchg && d->ctrl,
          B200_ERR_ARG);
  REQUIRE(d->L > 0 && d->H > 0 && d->I > 0 && d->n_q > 0 && d->n_kv > 0 && d->V > 0 && d->grid > 0 && d->ctx_cap > 0,
          B200_ERR_ARG);
  REQUIRE(d->D == 64 || d->D == 128, B200_ERR_SHAPE);
  // the tile layout holds one (scale, zero) per row and 128 columns: group sizes are multiples of 128
  REQUIRE(d->n_q % d->n_kv == 0 && d->log2G >= 7 && d->log2G < 31 && d->log2P >= 0 && d->log2P < 16, B200_ERR_SHAPE);
  const int n_att = d->n_q * d->D, n_qkv = (d->n_q + 2 * d->n_kv) * d->D;
  const int Ks[3] = {d->H, n_att, d->I};
  int kmax = 0;
  for (int K : Ks) {
    REQUIRE(K % 128 == 0 && K % (1 << d->log2G) == 0, B200_ERR_SHAPE);
    kmax = K > kmax ? K : kmax;
  }
  REQUIRE(aligned16(d->emb) && aligned16(d->norm_f) && aligned16(d->w_head) && aligned16(d->xchg) &&
              aligned16(d->ctrl) && aligned16(d->layers),
          B200_ERR_ALIGN);
  REQUIRE(d->ctx_cap <= (1 << 20), B200_ERR_LIMIT);

  b200::StepParams p = {};
  p.layers = reinterpret_cast<const b200::StepLayer*>(d->layers);
  p.L = d->L; p.H = d->H; p.I = d->I; p.n_q = d->n_q; p.n_kv = d->n_kv; p.D = d->D; p.V = d->V;
  p.log2G = d->log2G; p.log2P = d->log2P; p.eps = d->eps;
  p.emb = (const half*)d->emb; p.norm_f = (const half*)d->norm_f; p.w_head = d->w_head; p.sz_head = d->sz_head;
  p.cos_t = d->cos_t; p.sin_t = d->sin_t; p.bt = d->bt; p.tok = d->tok; p.pos = d->pos; p.history = d->history;
  p.logits = (half*)d->logits; p.xchg = (uint32_t*)d->xchg; p.ctrl = (b200::StepCtrl*)d->ctrl;
  p.trace = d->trace;
  p.att_slices = b200::step_att_slices(d->grid, d->n_q);
  // shared-memory plan
  const int ncw = b200::decode_step_consumer_warps();
  const int resid_bytes = align_up(2 * d->H, 128);
  const int xin_bytes = align_up(2 * kmax, 128);             // two byte digits per activation, as B fragments
  const int xsum_bytes = align_up((kmax / 128) * 8, 128);
  const int att_bytes = align_up((4 * d->D + ncw * d->D + 2 * ncw + d->D + 64) * 4, 128);
  int part_bytes;
  {
    // partial sums: one float per consumer warp and row slot of the CTA's tiles (16 slots per tile); the layer
    // phases alternate between two buffers, the LM head uses the same area as one
    auto tiles_per_cta = [&](int tiles) { return (tiles + d->grid - 1) / d->grid; };
    const int layer_tiles[4] = {(n_qkv + 15) / 16, (d->H + 15) / 16, (d->I + 7) / 8, (d->H + 15) / 16};
    int mt = 1;
    for (int t : layer_tiles) mt = tiles_per_cta(t) > mt ? tiles_per_cta(t) : mt;
    p.part_stride = 16 * mt + 1;                                      // odd pitch: the warps' rows start in
    p.part_stride_head = 16 * tiles_per_cta((d->V + 15) / 16) + 1;    // different banks
    const int a = 2 * ncw * p.part_stride, b = ncw * p.part_stride_head;
    part_bytes = align_up((a > b ? a : b) * 4, 128);
  }
  const int table_bytes = align_up(d->L * (int)sizeof(b200::StepLayer), 128);
  p.ups = B200_STEP_UPS;
  p.stage_w = p.ups * b200::kTileUnitBytes;
  p.stage_bytes = align_up(p.stage_w, 128);
  // attention copies whole KV pages into a stage, K rows in one half and V rows in the other
  const int P = 1 << d->log2P;
  REQUIRE(P <= b200::decode_step_max_kv_tokens() && 4 * d->D * P <= p.stage_w, B200_ERR_SHAPE);
  const size_t fixed = b200::decode_step_plan_smem(p, resid_bytes, xin_bytes, xsum_bytes, att_bytes, part_bytes,
                                                   table_bytes);
  const size_t budget = 227 * 1024;
  REQUIRE(fixed + 2 * (size_t)p.stage_bytes <= budget, B200_ERR_SHAPE);
  int ns = (int)((budget - fixed) / p.stage_bytes);
  if (ns > b200::decode_step_max_stages()) ns = b200::decode_step_max_stages();
  p.ns = ns;
  return finish(b200::decode_step_launch(p, d->grid, fixed + (size_t)ns * p.stage_bytes, S(stream)));
}

int b200_argmax(const void* logits, int V, long long* tok, int* pos, long long* history, void* stream) {
  REQUIRE(logits && tok && V > 0, B200_ERR_ARG);
  REQUIRE(history == nullptr || pos != nullptr, B200_ERR_ARG);
  return finish(b200::argmax_dispatch(logits, V, tok, pos, history, S(stream)));
}

// ---- tensor-parallel exchange blocks (the only entry points of the library that own device memory) -----------------
int b200_comm_header_bytes(void) { return b200::comm_header_bytes(); }

int b200_comm_alloc(size_t bytes, void** ptr) {
  REQUIRE(ptr && bytes >= (size_t)b200::comm_header_bytes(), B200_ERR_ARG);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    return finish(e);
  }
  *ptr = p;
  return B200_OK;
}

int b200_comm_free(void* ptr) {
  REQUIRE(ptr, B200_ERR_ARG);
  return finish(cudaFree(ptr));
}

int b200_comm_export(void* ptr, void* handle64) {
  REQUIRE(ptr && handle64, B200_ERR_ARG);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed around as 64 bytes");
  return finish(cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), ptr));
}

int b200_comm_import(const void* handle64, void** ptr) {
  REQUIRE(handle64 && ptr, B200_ERR_ARG);
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return finish(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}

int b200_comm_unimport(void* ptr) {
  REQUIRE(ptr, B200_ERR_ARG);
  return finish(cudaIpcCloseMemHandle(ptr));
}

int b200_comm_reset(void* base) {
  REQUIRE(base, B200_ERR_ARG);
  // flags, step counter and error word; the wait bound (b200_comm_set_wait_limit) is a setting and stays
  cudaError_t e = cudaMemset(base, 0, b200::comm_limit_offset());
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return finish(e);
}

int b200_comm_set_wait_limit(void* base, unsigned int polls) {
  REQUIRE(base, B200_ERR_ARG);
  cudaError_t e = cudaMemcpy((char*)base + b200::comm_limit_offset(), &polls, sizeof(polls), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  return finish(e);
}

int b200_comm_error(const void* base, int* code) {
  REQUIRE(base && code, B200_ERR_ARG);
  return finish(cudaMemcpy(code, (const char*)base + b200::comm_error_offset(), sizeof(int), cudaMemcpyDeviceToHost));
}

static int check_peers(const void* const* peers, int rank, int W, size_t off) {
  REQUIRE(peers && W >= 1 && W <= b200::comm_max_ranks() && rank >= 0 && rank < W, B200_ERR_ARG);
  REQUIRE(off >= (size_t)b200::comm_header_bytes() && off % 16 == 0, B200_ERR_ALIGN);
  for (int r = 0; r < W; ++r) REQUIRE(peers[r] && aligned16(peers[r]), B200_ERR_ARG);
  return B200_OK;
}

int b200_tp_allreduce_add_rmsnorm(const void* const* peers, int rank, int W, size_t slot_off, void* x, const void* w,
                                  void* out, int H, float eps, void* stream) {
  const int rc = check_peers(peers, rank, W, slot_off);
  if (rc) return rc;
  REQUIRE(x && w && out && H > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(H <= 32768, B200_ERR_LIMIT);
  REQUIRE(aligned16(x) && aligned16(w) && aligned16(out), B200_ERR_ALIGN);
  return finish(b200::tp_allreduce_add_rmsnorm_dispatch(peers, rank, W, slot_off, x, w, out, H, eps, S(stream)));
}

size_t b200_tp_gemv_slot_bytes(int N, int W) {
  if (N <= 0 || W < 1 || W > b200::comm_max_ranks()) return 0;
  return b200::gemv_allreduce_slot_bytes(N, W);
}

static int gemv_push_or_allreduce(const void* Wt, const void* x, void* y, int N, int K, const void* const* peers,
                                  int rank, int W, size_t slot_off, int tagged, void* stream) {
  REQUIRE(Wt && x && (y || tagged) && N > 0 && K > 0, B200_ERR_ARG);
  REQUIRE(K % 128 == 0 && N % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(K <= 65536, B200_ERR_LIMIT);
  REQUIRE(peers && W >= 1 && W <= b200::comm_max_ranks() && rank >= 0 && rank < W, B200_ERR_ARG);
  REQUIRE(slot_off >= (size_t)b200::comm_header_bytes() && slot_off % 256 == 0, B200_ERR_ALIGN);
  for (int r = 0; r < W; ++r) REQUIRE(peers[r] && aligned16(peers[r]), B200_ERR_ARG);
  REQUIRE(aligned16(Wt) && (reinterpret_cast<uintptr_t>(x) & 7u) == 0 && aligned16(y), B200_ERR_ALIGN);
  const cudaError_t e =
      b200::gemv_w4a16_tiled_allreduce_dispatch(Wt, x, y, N, K, peers, rank, W, slot_off, tagged, S(stream));
  if (e == cudaErrorInvalidValue) return B200_ERR_LIMIT;   // more thread blocks than the slot has flag rows
  return finish(e);
}

int b200_gemv_w4a16_tiled_allreduce(const void* Wt, const void* x, void* y, int N, int K, const void* const* peers,
                                    int rank, int W, size_t slot_off, void* stream) {
  return gemv_push_or_allreduce(Wt, x, y, N, K, peers, rank, W, slot_off, 0, stream);
}

int b200_gemv_w4a16_tiled_push(const void* Wt, const void* x, int N, int K, const void* const* peers, int rank, int W,
                               size_t slot_off, void* stream) {
  return gemv_push_or_allreduce(Wt, x, nullptr, N, K, peers, rank, W, slot_off, 1, stream);
}

int b200_tp_pushed_add_rmsnorm(const void* const* peers, int rank, int W, size_t slot_off, void* x, const void* w,
                               void* out, int H, float eps, void* stream) {
  REQUIRE(peers && W >= 1 && W <= b200::comm_max_ranks() && rank >= 0 && rank < W, B200_ERR_ARG);
  REQUIRE(slot_off >= (size_t)b200::comm_header_bytes() && slot_off % 256 == 0, B200_ERR_ALIGN);
  REQUIRE(peers[rank] && aligned16(peers[rank]), B200_ERR_ARG);
  REQUIRE(x && w && out && H > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(H <= 32768, B200_ERR_LIMIT);
  REQUIRE(aligned16(x) && aligned16(w) && aligned16(out), B200_ERR_ALIGN);
  return finish(b200::tp_pushed_add_rmsnorm_dispatch(peers, rank, W, slot_off, x, w, out, H, eps, S(stream)));
}

int b200_tp_allgather(const void* const* peers, int rank, int W, size_t slot_off, void* dst, int n, void* stream) {
  const int rc = check_peers(peers, rank, W, slot_off);
  if (rc) return rc;
  REQUIRE(dst && n > 0, B200_ERR_ARG);
  REQUIRE(n % 8 != 0 || aligned16(dst), B200_ERR_ALIGN);
  return finish(b200::tp_allgather_dispatch(peers, rank, W, slot_off, dst, n, S(stream)));
}

}  // extern "C"
