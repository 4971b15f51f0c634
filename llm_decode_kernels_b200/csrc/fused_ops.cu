// The small operators of the decode step: residual add + RMSNorm, SwiGLU, RoPE + paged KV append, embedding
// row fetch, greedy argmax, and the read-bandwidth probe. Each is a vector of a few KB, so launch latency
// and the number of dependent memory round trips matter, not bandwidth: every kernel makes one pass with the
// data held in registers between its phases.
#include "common.cuh"
#include <math_constants.h>

namespace b200 {

// ---- residual add + RMSNorm -----------------------------------------------------------------------------
// Replaces add_rmsnorm_launch (reference kernels/fused_norm.cu:56-58). Rounding as in HF LlamaRMSNorm
// (reference reference/ref_ops.py:15-20): x <- x +_fp16 delta (written back); h = half(float(x) * rsqrt(
// mean(float(x)^2) + eps)); out = w *_fp16 h. One block; each thread keeps its 8-element chunks in
// registers across the reduction, so x is read once. With a batch (the prompt's tokens) block b takes row b.
constexpr int kNormThreads = 512;
constexpr int kNormMaxChunks = 8;  // H <= 512 * 8 * 8 = 32768

__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_kernel(half* __restrict__ x, const half* __restrict__ delta, const half* __restrict__ w,
                   half* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  x += (size_t)blockIdx.x * H;
  out += (size_t)blockIdx.x * H;
  if (delta) delta += (size_t)blockIdx.x * H;
  __shared__ float part[kNormThreads / 32];
  const int tid = threadIdx.x, nchunk = H >> 3;
  uint4 xv[kNormMaxChunks];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = tid + c * kNormThreads;
    if (i < nchunk) {
      uint4 v = reinterpret_cast<const uint4*>(x)[i];
      if (delta) {
        const uint4 d = reinterpret_cast<const uint4*>(delta)[i];
        v.x = as_u32(__hadd2(as_h2(v.x), as_h2(d.x)));
        v.y = as_u32(__hadd2(as_h2(v.y), as_h2(d.y)));
        v.z = as_u32(__hadd2(as_h2(v.z), as_h2(d.z)));
        v.w = as_u32(__hadd2(as_h2(v.w), as_h2(d.w)));
        reinterpret_cast<uint4*>(x)[i] = v;
      }
      float f[8];
      unpack8(v, f);
#pragma unroll
      for (int k = 0; k < 8; ++k) ss = fmaf(f[k], f[k], ss);
      xv[c] = v;
    }
  }
  ss = warp_sum(ss);
  if ((tid & 31) == 0) part[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < kNormThreads / 32; ++k) tot += part[k];
  const float r = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int c = 0; c < kNormMaxChunks; ++c) {
    const int i = tid + c * kNormThreads;
    if (i < nchunk) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + i);
      const uint32_t xu[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(as_h2(xu[k]));
        o[k] = as_u32(__hmul2(as_h2(wu[k]), __floats2half2_rn(f.x * r, f.y * r)));
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

cudaError_t add_rmsnorm_dispatch(void* x, const void* delta, const void* w, void* out, int rows, int H, float eps,
                                 cudaStream_t st) {
  B200_LAUNCH(add_rmsnorm_kernel, dim3(rows), dim3(kNormThreads), 0, st, (half*)x, (const half*)delta, (const half*)w,
              (half*)out, H, eps);
  return cudaPeekAtLastError();
}

// ---- SwiGLU ---------------------------------------------------------------------------------------------
// Replaces swiglu_launch (reference kernels/fused_swiglu.cu:23-26). gu = gate followed by up, [2I];
// out[i] = half(silu_fp32(gate_i)) *_fp16 up_i (reference reference/ref_ops.py:23-27). blockIdx.y = row of a batch
// (gu [rows, 2I], out [rows, I]).
__global__ void swiglu_kernel(const uint4* __restrict__ gate, const uint4* __restrict__ up, uint4* __restrict__ out,
                              int nchunk) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nchunk) return;
  gate += (size_t)blockIdx.y * 2 * nchunk;
  up += (size_t)blockIdx.y * 2 * nchunk;
  out += (size_t)blockIdx.y * nchunk;
  const uint4 gv = gate[i], uv = up[i];
  const uint32_t g[4] = {gv.x, gv.y, gv.z, gv.w}, u[4] = {uv.x, uv.y, uv.z, uv.w};
  uint32_t o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 f = __half22float2(as_h2(g[k]));
    const half2 s = __floats2half2_rn(f.x / (1.f + expf(-f.x)), f.y / (1.f + expf(-f.y)));
    o[k] = as_u32(__hmul2(s, as_h2(u[k])));
  }
  out[i] = make_uint4(o[0], o[1], o[2], o[3]);
}

cudaError_t swiglu_dispatch(const void* gu, void* out, int rows, int I, cudaStream_t st) {
  const int nchunk = I >> 3, threads = 128;
  B200_LAUNCH(swiglu_kernel, dim3((nchunk + threads - 1) / threads, rows), dim3(threads), 0, st, (const uint4*)gu, (const
              uint4*)((const half*)gu + I), (uint4*)out, nchunk);
  return cudaPeekAtLastError();
}

// ---- RoPE + paged KV append -----------------------------------------------------------------------------
// Replaces rope_append_launch (reference kernels/rope_kv.cu:34-38), generalised from head_dim 64 to any even D
// and to a batch of sequences. qkv [B, (n_q + 2 n_kv) D]; q is rotated in place, rotated k and untouched v
// go to page bt[b, pos_b / P], slot pos_b % P of caches laid out [pages, n_kv, P, D]. cos/sin fp32
// [max_pos, D/2]; pairs are (i, i + D/2) (reference reference/ref_ops.py:36-53). One block per head,
// one thread per pair.
__global__ void rope_append_kernel(half* __restrict__ qkv, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, const int* __restrict__ pos_ptr,
                                   const int* __restrict__ bt, int bt_stride, half* __restrict__ kc,
                                   half* __restrict__ vc, int n_q, int n_kv, int D, int log2P) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, b = blockIdx.y, i = threadIdx.x, d2 = D >> 1;
  const int pos = pos_ptr[b];
  half* v = qkv + ((size_t)b * (n_q + 2 * n_kv) + head) * D;
  const int page = bt[(size_t)b * bt_stride + (pos >> log2P)], slot = pos & ((1 << log2P) - 1);
  if (head < n_q + n_kv) {
    const float c = cos_t[(size_t)pos * d2 + i], s = sin_t[(size_t)pos * d2 + i];
    const float a = __half2float(v[i]), bb = __half2float(v[i + d2]);
    const half ra = __float2half(a * c - bb * s), rb = __float2half(bb * c + a * s);
    half* dst = head < n_q ? v : kc + ((((size_t)page * n_kv + (head - n_q)) << log2P) + slot) * D;
    dst[i] = ra;
    dst[i + d2] = rb;
  } else {
    half* dst = vc + ((((size_t)page * n_kv + (head - n_q - n_kv)) << log2P) + slot) * D;
    dst[i] = v[i];
    dst[i + d2] = v[i + d2];
  }
}

cudaError_t rope_append_dispatch(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                                 int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                                 cudaStream_t st) {
  B200_LAUNCH(rope_append_kernel, dim3(n_q + 2 * n_kv, B), dim3(D / 2), 0, st, (half*)qkv, cos_t, sin_t, pos, bt,
              bt_stride, (half*)kc, (half*)vc, n_q, n_kv, D, log2P);
  return cudaPeekAtLastError();
}

// ---- embedding row fetch: x[H] = emb[tok[0], :] (tok is int64 on the device) ------------------------------
// Stands in for the torch.index_select of the reference's step (runtime/model.py:218).
// A token id outside [0, V) must not become an address (the id comes from device memory: a caller's mistake or a
// corrupted step would otherwise read far outside the table); row 0 is copied instead.
__global__ void embed_row_kernel(const uint4* __restrict__ emb, const long long* __restrict__ tok,
                                 uint4* __restrict__ x, int nchunk, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  long long t = tok[0];
  if (t < 0 || t >= V) t = 0;
  if (i < nchunk) x[i] = emb[(size_t)t * nchunk + i];
}

cudaError_t embed_row_dispatch(const void* emb, const long long* tok, void* x, int H, int V, cudaStream_t st) {
  const int nchunk = H >> 3;
  B200_LAUNCH(embed_row_kernel, dim3((nchunk + 255) / 256), dim3(256), 0, st, (const uint4*)emb, tok, (uint4*)x,
              nchunk, V);
  return cudaPeekAtLastError();
}

// ---- greedy argmax over fp16 logits; lowest index wins ties; optionally advances pos -----------------------
// Stands in for torch.argmax + `pos += 1` at the end of the reference's step (runtime/model.py:232-233).
// With `history`, the chosen token is also stored at history[pos before the increment], so a run of graph
// replays leaves its whole token stream on the device and the host need not read a token per step.
// One block of 1024 threads; the order key packs (value, inverted index) so one max-reduction settles ties.
__global__ void __launch_bounds__(1024)
argmax_kernel(const half* __restrict__ logits, int V, long long* __restrict__ tok, int* __restrict__ pos,
              long long* __restrict__ history) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ unsigned long long part[32];
  unsigned long long best = 0ull;
  auto take = [&](half v, int i) {
    if (!__hisnan(v)) {
      const unsigned long long k = argmax_key(v, i);
      best = k > best ? k : best;
    }
  };
  // 16-byte loads (8 logits) where the vector allows, all of a thread's loads independent of each other: a 128 K
  // vocabulary is 16 loads per thread instead of 125 dependent-looking 2-byte ones. The key order settles ties, so the
  // order of the scan does not matter.
  const int nvec = (reinterpret_cast<uintptr_t>(logits) & 15u) == 0 ? V >> 3 : 0;
#pragma unroll 4
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    const uint4 u = reinterpret_cast<const uint4*>(logits)[c];
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const half2 h = as_h2(w[k]);
      take(__low2half(h), 8 * c + 2 * k);
      take(__high2half(h), 8 * c + 2 * k + 1);
    }
  }
  for (int i = 8 * nvec + threadIdx.x; i < V; i += blockDim.x) take(logits[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
    best = other > best ? other : best;
  }
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    best = part[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
    if (threadIdx.x == 0) {
      // best == 0: no comparable logit (all NaN). torch.argmax, which the reference uses, still answers with a valid
      // index; token 0 is this kernel's answer, so the next step's embedding read stays inside the table.
      const long long t = best ? (long long)(0x7FFFFFFF - (int)(best & 0xFFFFFFFFu)) : 0ll;
      tok[0] = t;
      if (pos) {
        const int p = pos[0];
        if (history) history[p] = t;  // the token predicted after consuming position p
        pos[0] = p + 1;
      }
    }
  }
}

cudaError_t argmax_dispatch(const void* logits, int V, long long* tok, int* pos, long long* history,
                            cudaStream_t st) {
  B200_LAUNCH(argmax_kernel, dim3(1), dim3(1024), 0, st, (const half*)logits, V, tok, pos, history);
  return cudaPeekAtLastError();
}

// ---- read-bandwidth probe -------------------------------------------------------------------------------
// Replaces bw_read_launch (reference kernels/gemv_w4a16.cu:149-153): XOR-reduces a buffer with the same
// streaming loads the GEMV uses; the achieved GB/s is this library's own "achievable HBM read" figure.
template <int UNROLL>
__global__ void bw_read_kernel(const uint4* __restrict__ p, size_t n, uint32_t* sink) {
  uint32_t a = 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (UNROLL - 1) * stride < n; i += UNROLL * stride) {
    uint4 v[UNROLL];
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) v[k] = ld_stream(p + i + k * stride);
#pragma unroll
    for (int k = 0; k < UNROLL; ++k) a ^= v[k].x ^ v[k].y ^ v[k].z ^ v[k].w;
  }
  for (; i < n; i += stride) {
    const uint4 v = ld_stream(p + i);
    a ^= v.x ^ v.y ^ v.z ^ v.w;
  }
  if (a == 0x5bd1e995u) *sink = a;  // keeps the loads alive; practically never true
}

cudaError_t bw_read_dispatch(const void* p, size_t bytes, void* sink, int blocks, int threads, int unroll,
                             cudaStream_t st) {
  const size_t n = bytes / 16;
  if (unroll >= 8) bw_read_kernel<8><<<blocks, threads, 0, st>>>((const uint4*)p, n, (uint32_t*)sink);
  else if (unroll >= 4) bw_read_kernel<4><<<blocks, threads, 0, st>>>((const uint4*)p, n, (uint32_t*)sink);
  else bw_read_kernel<1><<<blocks, threads, 0, st>>>((const uint4*)p, n, (uint32_t*)sink);
  return cudaPeekAtLastError();
}

}  // namespace b200

// ---- read-bandwidth probe through a bulk-copy ring -------------------------------------------------------------
// Same question as bw_read, asked of the path the persistent step kernel uses: one elected thread per CTA streams
// the CTA's share of the buffer into a shared-memory ring with cp.async.bulk (mbarrier transaction counts), the
// other warps touch one word of every stage and release it. Waits are bounded: a wait that runs out sets *sink to
// 0xdead0000 + code and the CTA stops.
namespace b200 {
namespace {
DEVI uint32_t probe_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI bool probe_wait(uint64_t* bar, uint32_t parity) {
  for (int i = 0; i < (1 << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(probe_smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
}  // namespace

__global__ void __launch_bounds__(160, 1)
bw_read_bulk_kernel(const uint8_t* __restrict__ p, size_t bytes, uint32_t* sink, int stage_bytes, int ns) {
  extern __shared__ __align__(128) uint8_t ring_smem[];
  uint64_t* full = reinterpret_cast<uint64_t*>(ring_smem);
  uint64_t* empty = full + 32;
  uint8_t* ring = ring_smem + 512;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int i = 0; i < ns; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(probe_smem_u32(&full[i])), "r"(1));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(probe_smem_u32(&empty[i])), "r"(4));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const size_t nstage_total = bytes / stage_bytes;
  const size_t per = nstage_total / gridDim.x;           // stages per CTA (remainder ignored)
  const uint8_t* src = p + (size_t)blockIdx.x * per * stage_bytes;
  if (warp == 4) {
    if (lane == 0) {
      for (size_t it = 0; it < per; ++it) {
        const int slot = (int)(it % ns);
        if (!probe_wait(&empty[slot], (uint32_t)(((it / ns) & 1) ^ 1))) { *sink = 0xdead0003u; return; }
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(probe_smem_u32(&full[slot])),
                     "r"(stage_bytes)
                     : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         probe_smem_u32(ring + (size_t)slot * stage_bytes)),
                     "l"(src + it * stage_bytes), "r"(stage_bytes), "r"(probe_smem_u32(&full[slot]))
                     : "memory");
      }
    }
    return;
  }
  uint32_t a = 0;
  for (size_t it = 0; it < per; ++it) {
    const int slot = (int)(it % ns);
    if (!probe_wait(&full[slot], (uint32_t)((it / ns) & 1))) { *sink = 0xdead0002u; return; }
    a ^= reinterpret_cast<const uint32_t*>(ring + (size_t)slot * stage_bytes)[tid];
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(probe_smem_u32(&empty[slot])) : "memory");
  }
  if (a == 0x5bd1e995u) *sink = a;
}

cudaError_t bw_read_bulk_dispatch(const void* p, size_t bytes, void* sink, int blocks, int stage_bytes, int stages,
                                  cudaStream_t st) {
  const size_t smem = 512 + (size_t)stage_bytes * stages;
  cudaError_t e = cudaFuncSetAttribute(bw_read_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
  if (e != cudaSuccess) return e;
  bw_read_bulk_kernel<<<blocks, 160, smem, st>>>((const uint8_t*)p, bytes, (uint32_t*)sink, stage_bytes, stages);
  return cudaPeekAtLastError();
}
}  // namespace b200
