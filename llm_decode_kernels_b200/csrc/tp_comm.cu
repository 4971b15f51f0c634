// Tensor-parallel exchange over NVLink peer memory, fused with the operator that follows it.
//
// A row-split projection (o_proj, down_proj) leaves every rank with a partial [H] vector; the reference design for
// the 70B shape sums them with an NCCL all-reduce and then runs residual add + RMSNorm. Here each rank's GEMV writes
// its partial straight into a buffer that the other GPUs of the node can read (CUDA IPC mapping, one process per
// GPU), and ONE kernel per rank does the rest:
//   1. tell every peer "my partial number `step` is ready" (a release store of `step` into the peer's flag word),
//   2. wait until every peer has said the same (acquire loads of the local flag words, bounded),
//   3. read all W partials (peer loads over NVLink), add them in rank order with fp32 accumulation - the same order
//      on every rank, so all ranks compute bit-identical sums -, round to fp16,
//   4. residual add and RMSNorm exactly as add_rmsnorm_kernel does.
// That is a one-shot all-reduce: for 16 KB vectors latency is everything, and one round of flag + data over NVSwitch
// is the least it can cost. No library kernel touches peer memory, nothing here uses multicast loads.
//
// The vocabulary-split LM head ends with the same flag round followed by a gather of the logit shards.
//
// Buffer reuse needs no second flag round: a rank signals step s+1 only after it has finished reading step s, and
// two buffers alternate (o_proj partials use one slot, down_proj partials another), so when a rank overwrites a slot
// every peer has signalled a later step and is therefore done with the slot's previous contents.
//
// Every wait is bounded (about four seconds by default, enough for ranks that drift apart between host-driven
// steps; a caller may store a shorter bound in the block's header). A wait that runs out stores a code in the
// block's error word, and the kernel returns without touching the outputs.
#include "tp_comm.cuh"

namespace b200 {

namespace {

// Steps 1 and 2 of the header comment, by all threads of the (single) block. Returns false if a wait ran out.
DEVI bool exchange_flags(const CommPeers& P, int rank, int W) {
  __shared__ uint32_t step_s;
  uint8_t* base = P.p[rank];
  const int tid = threadIdx.x;
  if (tid == 0) {
    uint32_t* counter = reinterpret_cast<uint32_t*>(base + kCommCounterOff);
    step_s = *counter + 1u;
    *counter = step_s;
  }
  __syncthreads();
  const uint32_t step = step_s;
  const uint32_t set_limit = *reinterpret_cast<const uint32_t*>(base + kCommLimitOff);
  const int limit = set_limit ? (int)set_limit : kCommSpinLimit;
  int failed = 0;
  if (tid < W && tid != rank) {
    __threadfence_system();   // the partial was written by the previous kernel of this stream; order it before the flag
    st_release_sys(reinterpret_cast<uint32_t*>(P.p[tid] + kCommFlagsOff) + rank, step);
    const uint32_t* mine = reinterpret_cast<const uint32_t*>(base + kCommFlagsOff) + tid;
    int i = 0;
    while ((int32_t)(ld_acquire_sys(mine) - step) < 0) {
      if (++i > limit) { failed = 1; break; }
      if (i > 256) __nanosleep(500);   // peers normally answer within microseconds: poll hard first, then back off
    }
    if (failed) atomicExch(reinterpret_cast<uint32_t*>(base + kCommErrorOff), COMM_ERR_PEER_WAIT);
  }
  return __syncthreads_or(failed) == 0;
}

}  // namespace

// delta = sum over ranks of the partial at `off` (fp32 accumulation in rank order, rounded to fp16), then
// x <- x +_fp16 delta, out <- w *_fp16 half(float(x) * rsqrt(mean(x^2) + eps)): the rounding of add_rmsnorm_kernel.
// One block of 1024 threads; H % 8 == 0, H <= 1024 * 8 * 4.
__global__ void __launch_bounds__(kCommThreads)
tp_allreduce_add_rmsnorm_kernel(const CommPeers P, int rank, int W, size_t off, half* __restrict__ x,
                                const half* __restrict__ w, half* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MAXC = 4;
  __shared__ float part[kCommThreads / 32];
  if (!exchange_flags(P, rank, W)) return;
  const int tid = threadIdx.x, nchunk = H >> 3;
  uint4 xv[MAXC];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i = tid + c * kCommThreads;
    if (i < nchunk) {
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      // all peers' pieces are requested before the first is used: one NVLink round trip instead of W
      for (int r0 = 0; r0 < W; r0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (r0 + j < W) v[j] = ld_peer16(P.p[r0 + j] + off + 16 * (size_t)i);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          if (r0 + j < W) {
            float f[8];
            unpack8(v[j], f);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += f[k];
          }
        }
      }
      uint4 v = reinterpret_cast<const uint4*>(x)[i];
      v.x = as_u32(__hadd2(as_h2(v.x), __floats2half2_rn(acc[0], acc[1])));
      v.y = as_u32(__hadd2(as_h2(v.y), __floats2half2_rn(acc[2], acc[3])));
      v.z = as_u32(__hadd2(as_h2(v.z), __floats2half2_rn(acc[4], acc[5])));
      v.w = as_u32(__hadd2(as_h2(v.w), __floats2half2_rn(acc[6], acc[7])));
      reinterpret_cast<uint4*>(x)[i] = v;
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
  for (int k = 0; k < kCommThreads / 32; ++k) tot += part[k];
  const float rinv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i = tid + c * kCommThreads;
    if (i < nchunk) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + i);
      const uint32_t xu[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(as_h2(xu[k]));
        o[k] = as_u32(__hmul2(as_h2(wu[k]), __floats2half2_rn(f.x * rinv, f.y * rinv)));
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// The consumer of a GEMV that pushed tagged words (gemv_w4a16.cu, ALLRED epilogue, tagged form): every rank's rows of
// this call lie - or are about to arrive - in THIS rank's slot as words (tag << 16 | fp16). Poll them until they carry
// the call's tag (bounded), add the W copies in rank order with fp32 accumulation, round to fp16, then residual add
// and RMSNorm as add_rmsnorm_kernel does. No flag, no fence, no peer load: the exchange costs one NVLink flight after
// the producers' last store. The call counter of the slot moves on when the block is done reading.
// One block of 1024 threads; H % 8 == 0, H <= 1024 * 8 * 4. On a timeout: error word, outputs untouched.
__global__ void __launch_bounds__(kCommThreads)
tp_pushed_add_rmsnorm_kernel(const CommPeers P, int rank, int W, size_t off, half* __restrict__ x,
                             const half* __restrict__ w, half* __restrict__ out, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MAXC = 4;
  __shared__ float part[kCommThreads / 32];
  __shared__ uint32_t call_s;
  uint8_t* base = P.p[rank];
  uint32_t* ctrl = reinterpret_cast<uint32_t*>(base + off);
  const int tid = threadIdx.x, nchunk = H >> 3;
  if (tid == 0) call_s = *reinterpret_cast<volatile uint32_t*>(ctrl) + 1u;
  __syncthreads();
  const uint32_t tagw = comm_tag(call_s);
  const uint32_t set_limit = *reinterpret_cast<const uint32_t*>(base + kCommLimitOff);
  const int limit = set_limit ? (int)set_limit : kCommSpinLimit;
  const uint8_t* data = base + off + kGemvSlotCtrlBytes + kGemvSlotFlagBytes;
  uint4 dsum[MAXC];   // the summed rows of this thread's chunks, already rounded to fp16
  int failed = 0;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i = tid + c * kCommThreads;
    dsum[c] = make_uint4(0u, 0u, 0u, 0u);
    if (i < nchunk && !failed) {
      float acc[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
      for (int r0 = 0; r0 < W && !failed; r0 += 2) {   // two ranks' pieces (four 16-byte loads) in flight together
        uint4 v[2][2];
        auto fetch = [&](int j) {
          const uint8_t* src = data + ((size_t)(r0 + j) * H + 8 * (size_t)i) * 4;
          v[j][0] = ld_peer16(src);
          v[j][1] = ld_peer16(src + 16);
        };
        auto fresh = [&](int j) {
          return ((((v[j][0].x ^ tagw) | (v[j][0].y ^ tagw) | (v[j][0].z ^ tagw) | (v[j][0].w ^ tagw) |
                    (v[j][1].x ^ tagw) | (v[j][1].y ^ tagw) | (v[j][1].z ^ tagw) | (v[j][1].w ^ tagw)) >> 16) == 0);
        };
#pragma unroll
        for (int j = 0; j < 2; ++j)
          if (r0 + j < W) fetch(j);
        int spins = 0;
        for (;;) {
          bool ok = true;
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (r0 + j < W && !fresh(j)) ok = false;
          if (ok) break;
          if (++spins > limit) { failed = 1; break; }
          if (spins > 256) __nanosleep(200);
#pragma unroll
          for (int j = 0; j < 2; ++j)
            if (r0 + j < W && !fresh(j)) fetch(j);
        }
        if (!failed) {
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (r0 + j < W) {
              const uint32_t wd[8] = {v[j][0].x, v[j][0].y, v[j][0].z, v[j][0].w,
                                      v[j][1].x, v[j][1].y, v[j][1].z, v[j][1].w};
#pragma unroll
              for (int k = 0; k < 8; ++k) acc[k] += __half2float(__ushort_as_half((unsigned short)(wd[k] & 0xFFFFu)));
            }
          }
        }
      }
      dsum[c].x = as_u32(__floats2half2_rn(acc[0], acc[1]));
      dsum[c].y = as_u32(__floats2half2_rn(acc[2], acc[3]));
      dsum[c].z = as_u32(__floats2half2_rn(acc[4], acc[5]));
      dsum[c].w = as_u32(__floats2half2_rn(acc[6], acc[7]));
    }
  }
  if (failed) atomicExch(reinterpret_cast<uint32_t*>(base + kCommErrorOff), COMM_ERR_PEER_WAIT);
  if (__syncthreads_or(failed)) return;   // every thread has its rows, or nobody writes anything
  if (tid == 0) *reinterpret_cast<volatile uint32_t*>(ctrl) = call_s;   // the slot may be pushed into again
  uint4 xv[MAXC];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i = tid + c * kCommThreads;
    if (i < nchunk) {
      uint4 v = reinterpret_cast<const uint4*>(x)[i];
      v.x = as_u32(__hadd2(as_h2(v.x), as_h2(dsum[c].x)));
      v.y = as_u32(__hadd2(as_h2(v.y), as_h2(dsum[c].y)));
      v.z = as_u32(__hadd2(as_h2(v.z), as_h2(dsum[c].z)));
      v.w = as_u32(__hadd2(as_h2(v.w), as_h2(dsum[c].w)));
      reinterpret_cast<uint4*>(x)[i] = v;
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
  for (int k = 0; k < kCommThreads / 32; ++k) tot += part[k];
  const float rinv = rsqrtf(tot / (float)H + eps);
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    const int i = tid + c * kCommThreads;
    if (i < nchunk) {
      const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + i);
      const uint32_t xu[4] = {xv[c].x, xv[c].y, xv[c].z, xv[c].w}, wu[4] = {wv.x, wv.y, wv.z, wv.w};
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(as_h2(xu[k]));
        o[k] = as_u32(__hmul2(as_h2(wu[k]), __floats2half2_rn(f.x * rinv, f.y * rinv)));
      }
      reinterpret_cast<uint4*>(out)[i] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// dst[r * n + i] = rank r's shard[i] (shards of n fp16 values at `off` of every block). One block of 1024 threads.
__global__ void __launch_bounds__(kCommThreads)
tp_allgather_kernel(const CommPeers P, int rank, int W, size_t off, half* __restrict__ dst, int n) {
  pdl_launch_dependents();
  pdl_wait();
  if (!exchange_flags(P, rank, W)) return;
  const int tid = threadIdx.x;
  if ((n & 7) == 0) {
    const int nchunk = n >> 3;
    for (int r = 0; r < W; ++r) {
      uint4* d = reinterpret_cast<uint4*>(dst + (size_t)r * n);
      const uint8_t* s = P.p[r] + off;
#pragma unroll 4
      for (int i = tid; i < nchunk; i += kCommThreads) d[i] = ld_peer16(s + 16 * (size_t)i);
    }
  } else {
    for (int r = 0; r < W; ++r) {
      const volatile half* s = reinterpret_cast<const volatile half*>(P.p[r] + off);
      for (int i = tid; i < n; i += kCommThreads) {
        const unsigned short u = reinterpret_cast<const volatile unsigned short*>(s)[i];
        dst[(size_t)r * n + i] = __ushort_as_half(u);
      }
    }
  }
}

cudaError_t tp_allreduce_add_rmsnorm_dispatch(const void* const* peers, int rank, int W, size_t off, void* x,
                                              const void* w, void* out, int H, float eps, cudaStream_t st) {
  CommPeers P = {};
  for (int r = 0; r < W; ++r) P.p[r] = (uint8_t*)peers[r];
  B200_LAUNCH(tp_allreduce_add_rmsnorm_kernel, dim3(1), dim3(kCommThreads), 0, st, P, rank, W, off, (half*)x, (const
              half*)w, (half*)out, H, eps);
  return cudaPeekAtLastError();
}

cudaError_t tp_pushed_add_rmsnorm_dispatch(const void* const* peers, int rank, int W, size_t off, void* x, const void* w,
                                           void* out, int H, float eps, cudaStream_t st) {
  CommPeers P = {};
  for (int r = 0; r < W; ++r) P.p[r] = (uint8_t*)peers[r];
  B200_LAUNCH(tp_pushed_add_rmsnorm_kernel, dim3(1), dim3(kCommThreads), 0, st, P, rank, W, off, (half*)x, (const
              half*)w, (half*)out, H, eps);
  return cudaPeekAtLastError();
}

cudaError_t tp_allgather_dispatch(const void* const* peers, int rank, int W, size_t off, void* dst, int n,
                                  cudaStream_t st) {
  CommPeers P = {};
  for (int r = 0; r < W; ++r) P.p[r] = (uint8_t*)peers[r];
  B200_LAUNCH(tp_allgather_kernel, dim3(1), dim3(kCommThreads), 0, st, P, rank, W, off, (half*)dst, n);
  return cudaPeekAtLastError();
}

int comm_header_bytes() { return kCommHeaderBytes; }
int comm_max_ranks() { return kCommMaxRanks; }
int comm_error_offset() { return kCommErrorOff; }
int comm_limit_offset() { return kCommLimitOff; }

}  // namespace b200
