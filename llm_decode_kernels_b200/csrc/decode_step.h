// Parameter block of the persistent decode-step kernel (decode_step.cu), shared with the C ABI (c_api.cu).
#pragma once
#include <cuda_fp16.h>
#include <stddef.h>
#include <stdint.h>

namespace b200 {

// One decoder layer; an array of these lives in DEVICE memory. Matrix order: 0 qkv, 1 o, 2 gate|up, 3 down.
// Bit-compatible with b200_step_layer of include/b200decode.h.
struct StepLayer {
  const void* w[4];    // packed int4 [N, K/8] int32
  const void* sz[4];   // (scale, zero) half2 [N, K/G]
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
  long long* trace;   // optional [grid][16 + 16 L] phase timestamps (ns)
  int debug;          // bit 0: do not wait for exchange tags (results are garbage; for timing experiments)
  // shared-memory plan, computed on the host
  int resid_bytes, xin_bytes, xsum_bytes, att_bytes, part_bytes, table_bytes, stage_w, stage_bytes, ns;
};

size_t decode_step_smem_fixed(const StepParams& p);
int decode_step_threads();
int decode_step_max_stages();
int decode_step_consumer_warps();
cudaError_t decode_step_launch(const StepParams& p, int grid, size_t smem, cudaStream_t st);

}  // namespace b200
