// Parameter block of the persistent decode-step kernel (decode_step.cu), shared with the C ABI (c_api.cu).
#pragma once
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>

namespace b200 {

// One decoder layer; an array of these lives in DEVICE memory. Matrix order: 0 qkv, 1 o, 2 gate|up, 3 down.
// Bit-compatible with b200_step_layer of include/b200decode.h.
struct StepLayer {
  const void* w[4];    // the matrix in tile layout (gemv_tile_repack_kernel); gate|up in its paired form
  const void* sz[4];   // unused: the tile layout carries (scale, zero)
  const half* ln1;
  const half* ln2;
  half* kc;            // [pages, n_kv, P, D]
  half* vc;
};

// Device-resident control word block (16 bytes, zero-initialised by the caller).
struct StepCtrl {
  unsigned int epoch;  // completed steps; the tag of exchange words is derived from epoch + 1
  int error;           // 0, or the code of the first wait that gave up
  int abort;           // raised with error; makes every CTA leave
  int pad;
};

struct StepParams {
  const StepLayer* layers;
  int L, H, I, n_q, n_kv, D, V, log2G, log2P;
  float eps;
  const half* emb;
  const half* norm_f;
  const void* w_head;
  const void* sz_head;
  const float* cos_t;
  const float* sin_t;
  const int* bt;
  long long* tok;
  int* pos;
  long long* history;
  half* logits;
  uint32_t* xchg;
  StepCtrl* ctrl;
  long long* trace;   // [grid][8 + 25 (L + 1)] phase timestamps (ns); read only by builds with -DB200_STEP_TRACE
  // shared-memory plan, computed on the host: byte offsets of the areas behind the header and the residual stream
  int off_xin, off_xsum, off_att, off_part, off_table, off_ring;
  int ups;               // tile-unit blocks (kTileUnitBytes each) per ring stage
  int stage_w;           // bytes of a stage that carry data (= ups * kTileUnitBytes)
  int stage_bytes, ns;   // stage pitch and number of stages of the ring
  int part_stride;       // row slots per warp in a partial-sum buffer of the layer phases (two buffers)
  int part_stride_head;  // the same for the LM head (one buffer over the same area)
  int att_slices;        // J: context slices per query head in attention (step_att_slices)
};

// Attention of the step: query head h is worked on by J CTAs, slice j taking the ring stages j, j + J, ... of the
// cached context; J = as many as the grid has CTAs for, at most kStepMaxAttSlices. Each slice publishes a normalised
// partial output and its log-sum-exp (two fp16 words: value and remainder); the CTAs that stage the attention output
// for the o projection merge the J partials while they stage.
#ifndef B200_STEP_MAX_SLICES
#define B200_STEP_MAX_SLICES 4   // build-time knob for measurements: 1 = one CTA per query head
#endif
constexpr int kStepMaxAttSlices = B200_STEP_MAX_SLICES;
inline int step_att_slices(int grid, int n_q) {
  const int j = grid / n_q;
  return j < 1 ? 1 : (j > kStepMaxAttSlices ? kStepMaxAttSlices : j);
}
// exchange words per query head for the log-sum-exps: pairs (value, remainder) per slice, padded to whole granules
__host__ __device__ inline int step_lse_words(int J) { return (2 * J + 3) & ~3; }
// exchange words of one layer: qkv, J partial attention outputs, log-sum-exps, o, act, down
__host__ __device__ inline size_t step_words_per_layer(int H, int I, int n_q, int n_kv, int D, int J) {
  return (size_t)(n_q + 2 * n_kv) * D + (size_t)J * n_q * D + (size_t)n_q * step_lse_words(J) + H + I + H;
}

size_t decode_step_plan_smem(StepParams& p, int resid_bytes, int xin_bytes, int xsum_bytes, int att_bytes,
                             int part_bytes, int table_bytes);
int decode_step_threads();
int decode_step_max_stages();
int decode_step_consumer_warps();
int decode_step_max_kv_tokens();
cudaError_t decode_step_launch(const StepParams& p, int grid, size_t smem, cudaStream_t st);

}  // namespace b200
