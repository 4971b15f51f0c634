// extern "C" boundary of libb200decode.so: argument checks, then one dispatch per call. Declarations and the
// per-function contract are in include/b200decode.h. Checks mirror the ones the reference performs in its
// Python binding before launching (kernels/bindings.cpp:18-24, 29-35, 47-56, 66-69, 76-77, 84-85), so a bad call
// fails on the host with a code instead of faulting on the device.
#include "../../include/b200decode.h"
#include "common.cuh"

namespace b200 {
cudaError_t gemv_w4a16_dispatch(int stage, int R, int warps, const void* Wp, const void* SZ, const void* x, void* y,
                                int N, int K, int log2G, cudaStream_t st);
cudaError_t dequant_w4a16_dispatch(const void* Wp, const void* SZ, void* out, int N, int K, int log2G,
                                   cudaStream_t st);
cudaError_t add_rmsnorm_dispatch(void* x, const void* delta, const void* w, void* out, int H, float eps,
                                 cudaStream_t st);
cudaError_t swiglu_dispatch(const void* gu, void* out, int I, cudaStream_t st);
cudaError_t rope_append_dispatch(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                                 int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                                 cudaStream_t st);
cudaError_t embed_row_dispatch(const void* emb, const long long* tok, void* x, int H, cudaStream_t st);
cudaError_t argmax_dispatch(const void* logits, int V, long long* tok, int* pos, long long* history,
                            cudaStream_t st);
cudaError_t bw_read_dispatch(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll,
                             cudaStream_t st);
cudaError_t paged_attention_dispatch(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
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

int b200_bw_read(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll, void* stream) {
  REQUIRE(p && sink && bytes >= 16 && blocks > 0 && threads > 0 && threads <= 1024, B200_ERR_ARG);
  REQUIRE(aligned16(p), B200_ERR_ALIGN);
  return finish(b200::bw_read_dispatch(p, bytes, sink, blocks, threads, unroll, S(stream)));
}

int b200_paged_attention_batched(const void* q, const void* kc, const void* vc, const int* bt, int bt_stride,
                                 const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS, int max_splits,
                                 float* o_part, float* m_part, float* l_part, void* out, void* stream) {
  REQUIRE(q && kc && vc && bt && pos && out, B200_ERR_ARG);
  REQUIRE(B > 0 && B <= 65535 && n_q > 0 && n_kv > 0 && PS > 0 && max_splits > 0 && max_splits <= 65535 &&
              bt_stride > 0 && log2P >= 0 && log2P < 16,
          B200_ERR_ARG);
  REQUIRE(max_splits == 1 || (o_part && m_part && l_part), B200_ERR_ARG);
  REQUIRE(D == 64 || D == 128, B200_ERR_SHAPE);
  REQUIRE(n_q % n_kv == 0, B200_ERR_SHAPE);
  const int hpg = n_q / n_kv;
  REQUIRE(hpg == 1 || hpg == 2 || hpg == 4 || hpg == 8, B200_ERR_SHAPE);
  REQUIRE(aligned16(kc) && aligned16(vc), B200_ERR_ALIGN);
  return finish(b200::paged_attention_dispatch(q, kc, vc, bt, bt_stride, pos, B, n_q, n_kv, D, log2P, PS, max_splits,
                                               o_part, m_part, l_part, out, S(stream)));
}

int b200_paged_attention(int version, const void* q, const void* kc, const void* vc, const int* bt, const int* pos,
                         int n_q, int n_kv, int log2P, int PS, int max_splits, float* o_part, float* m_part,
                         float* l_part, void* out, void* stream) {
  REQUIRE(version >= 1 && version <= 3, B200_ERR_ARG);
  return b200_paged_attention_batched(q, kc, vc, bt, 1 << 30, pos, 1, n_q, n_kv, 64, log2P, PS, max_splits, o_part,
                                      m_part, l_part, out, stream);
}

int b200_add_rmsnorm(void* x, const void* delta, const void* w, void* out, int H, float eps, void* stream) {
  REQUIRE(x && w && out && H > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(H <= 32768, B200_ERR_LIMIT);
  REQUIRE(aligned16(x) && aligned16(w) && aligned16(out) && aligned16(delta), B200_ERR_ALIGN);
  return finish(b200::add_rmsnorm_dispatch(x, delta, w, out, H, eps, S(stream)));
}

int b200_swiglu(const void* gu, void* out, int I, void* stream) {
  REQUIRE(gu && out && I > 0, B200_ERR_ARG);
  REQUIRE(I % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(aligned16(gu) && aligned16(out), B200_ERR_ALIGN);
  return finish(b200::swiglu_dispatch(gu, out, I, S(stream)));
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

int b200_embed_row(const void* emb, const long long* tok, void* x, int H, void* stream) {
  REQUIRE(emb && tok && x && H > 0, B200_ERR_ARG);
  REQUIRE(H % 8 == 0, B200_ERR_SHAPE);
  REQUIRE(aligned16(emb) && aligned16(x), B200_ERR_ALIGN);
  return finish(b200::embed_row_dispatch(emb, tok, x, H, S(stream)));
}

int b200_argmax(const void* logits, int V, long long* tok, int* pos, long long* history, void* stream) {
  REQUIRE(logits && tok && V > 0, B200_ERR_ARG);
  REQUIRE(history == nullptr || pos != nullptr, B200_ERR_ARG);
  return finish(b200::argmax_dispatch(logits, V, tok, pos, history, S(stream)));
}

}  // extern "C"
