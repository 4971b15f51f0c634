// Batched W4A16 GEMM for the prompt:  Y[T, N] = X[T, K] . dequant(W)[N, K]^T, fp32 accumulation, fp16 out.
//
// The reference processes a prompt token by token through its decode step (runtime/model.py:267-276) and records its
// tensor-core prefill GEMM as cut (RESULTS.md:385-387). With T tokens at once every weight is read once instead of T
// times, and the product is a dense contraction - the one place in this library where the 5th-generation tensor cores
// fit: tcgen05.mma, operands in shared memory, accumulator in tensor memory.
//
// One CTA computes a 128-row block of W for all T tokens: D[128 features, T tokens] (+)= A[128, 64] . B[T, 64]^T per
// 64-column chunk of K, as four tcgen05.mma.kind::f16 of K = 16 each.
//   A = the weights: the CTA's threads read the packed words and the groups' (scale, zero), dequantize exactly as
//       dequant_w4a16_kernel does (so the fp16 weights are the format's, bit for bit) and store 16-byte pieces into
//       shared memory in the K-major 128-byte-swizzle layout the MMA's descriptor names;
//   B = the activations, fp16 rows of X, copied into the same layout (rows past T are zeros);
//   D = fp32 in tensor memory: 128 lanes (features) x T columns, allocated with tcgen05.alloc, read back with
//       tcgen05.ld by the warp that owns the 32 lanes, rounded to fp16 and stored to Y[token][feature].
// Two shared-memory stages: while the tensor core works on one chunk (tcgen05.commit arrives on an mbarrier when it
// has finished with the stage) the threads fill the other.
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word (b200_prefill_gemm_status), the CTA
// stops issuing, frees its tensor memory and returns.
#include "common.cuh"

namespace b200 {

namespace {

constexpr int kPfThreads = 128;        // 4 warps: one per 32 lanes of tensor memory
constexpr int kPfRows = 128;           // rows of W per CTA = M of the MMA
constexpr int kPfChunk = 64;           // K elements per stage: one 128-byte swizzle row of fp16
constexpr int kPfMaxT = 256;           // tokens per call = N of the MMA (multiple of 16)
constexpr int kPfSpinLimit = 1 << 22;

__device__ int g_prefill_status = 0;   // 0, or 1 once a bounded wait inside prefill_gemm_kernel ran out

DEVI uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

DEVI void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(count));
}
DEVI bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
DEVI bool mbar_wait_bounded(uint64_t* b, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < kPfSpinLimit; ++i)
    if (mbar_try_wait(b, parity)) return true;
  return false;
}

// Shared-memory matrix descriptor of a K-major operand tile in the 128-byte-swizzle layout: rows of 64 fp16 (128
// bytes), eight rows per 1024-byte block, 16-byte piece c of row r stored at piece c ^ (r % 8). Fields: start address
// / 16 in bits 0-13, leading-dimension byte offset / 16 in bits 16-29 (not used by swizzled K-major tiles: 1),
// stride between 8-row blocks / 16 in bits 32-45 (1024 bytes), descriptor version 1 in bits 46-47, layout type
// 2 = 128-byte swizzle in bits 61-63.
DEVI uint64_t umma_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor of tcgen05.mma.kind::f16: D fp32 (bits 4-5 = 1), A and B fp16 (bits 7-9, 10-12 = 0), both
// K-major (bits 15, 16 = 0), N / 8 in bits 17-22, M / 16 in bits 24-28.
DEVI uint32_t umma_idesc_f16(int M, int N) { return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24); }

DEVI void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
DEVI void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
               : "memory");
}

// byte offset of 16-byte piece c (0..7) of row r inside a swizzled tile
DEVI uint32_t sw128_offset(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

}  // namespace

// Wp int32 [N, K/8], SZ half2 [N, K >> log2G] (the quantizer's row-major tensors), X fp16 [T, K], Y fp16 [T, N].
// Tpad = T rounded up to a multiple of 16 (the MMA's N); K % 64 == 0; the group size a multiple of 64.
__global__ void __launch_bounds__(kPfThreads)
prefill_gemm_kernel(const uint32_t* __restrict__ Wp, const half2* __restrict__ SZ, const half* __restrict__ X,
                    half* __restrict__ Y, int T, int Tpad, int N, int K, int log2G, int tmem_cols) {
  extern __shared__ uint8_t pf_raw[];
  __shared__ __align__(8) uint64_t mma_done[2];
  __shared__ uint32_t tmem_base_s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~(uintptr_t)1023);
  const int a_bytes = kPfRows * 128, b_bytes = Tpad * 128;
  uint8_t* sA[2] = {base, base + a_bytes + b_bytes};
  uint8_t* sB[2] = {base + a_bytes, base + 2 * a_bytes + b_bytes};
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {   // one warp allocates the accumulator's columns of tensor memory for the CTA
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_s)),
                 "r"((uint32_t)tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    mbar_init(&mma_done[0], 1);
    mbar_init(&mma_done[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;

  const int row0 = blockIdx.x * kPfRows, words = K >> 3, ng = K >> log2G, nchunks = K / kPfChunk;
  const uint32_t idesc = umma_idesc_f16(kPfRows, Tpad);
  const half2 k1024 = __float2half2_rn(1024.f);
  bool failed = false;

  for (int i = 0; i < nchunks; ++i) {
    const int s = i & 1;
    if (i >= 2) {   // the MMAs that read this stage two chunks ago must have finished
      const int bad = mbar_wait_bounded(&mma_done[s], ((i >> 1) - 1) & 1) ? 0 : 1;
      if (__syncthreads_or(bad)) { failed = true; break; }
    }
    // A: 128 rows x 8 pieces; one piece = one packed word = 8 weights, dequantized as dequant_w4a16_kernel does
    for (int p = tid; p < kPfRows * 8; p += kPfThreads) {
      const int r = p >> 3, c = p & 7, row = row0 + r;
      uint4 o = make_uint4(0u, 0u, 0u, 0u);
      if (row < N) {
        const uint32_t w = __ldg(Wp + (size_t)row * words + i * 8 + c);
        const half2 sz = __ldg(SZ + (size_t)row * ng + ((i * kPfChunk + c * 8) >> log2G));
        const half2 s2 = __half2half2(__low2half(sz));
        const half2 zl = __hadd2(__half2half2(__high2half(sz)), k1024);
        o.x = as_u32(__hmul2(__hsub2(nib_lo(w), zl), s2));
        o.y = as_u32(__hmul2(__hsub2(nib_lo(w >> 4), zl), s2));
        o.z = as_u32(__hmul2(__hsub2(nib_lo(w >> 8), zl), s2));
        o.w = as_u32(__hmul2(__hsub2(nib_lo(w >> 12), zl), s2));
      }
      *reinterpret_cast<uint4*>(sA[s] + sw128_offset(r, c)) = o;
    }
    // B: Tpad token rows x 8 pieces of the activations
    for (int p = tid; p < Tpad * 8; p += kPfThreads) {
      const int t = p >> 3, c = p & 7;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (t < T) v = __ldg(reinterpret_cast<const uint4*>(X + (size_t)t * K + i * kPfChunk) + c);
      *reinterpret_cast<uint4*>(sB[s] + sw128_offset(t, c)) = v;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
    __syncthreads();
    if (tid == 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t da = umma_desc_sw128(smem_addr(sA[s])), db = umma_desc_sw128(smem_addr(sB[s]));
#pragma unroll
      for (int k = 0; k < kPfChunk / 16; ++k)   // 16 fp16 = 32 bytes further along the swizzled row: +2 in units of 16 B
        umma_f16(tmem, da + 2 * k, db + 2 * k, idesc, (i | k) != 0 ? 1u : 0u);
      umma_commit(&mma_done[s]);
    }
  }

  if (!failed) {   // the commit of the last chunk covers every MMA before it
    const int last = nchunks - 1;
    const int bad = mbar_wait_bounded(&mma_done[last & 1], (last >> 1) & 1) ? 0 : 1;
    failed = __syncthreads_or(bad) != 0;
  }
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (!failed) {
    // warp w owns lanes 32 w .. 32 w + 31 of tensor memory = features row0 + 32 w + lane; 16 token columns per load
    const int feature = row0 + 32 * warp + lane;
    for (int c0 = 0; c0 < Tpad; c0 += 16) {
      uint32_t v[16];
      const uint32_t taddr = tmem + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
          : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
            "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
          : "r"(taddr)
          : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (feature < N) {
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (c0 + j < T) Y[(size_t)(c0 + j) * N + feature] = __float2half(__uint_as_float(v[j]));
      }
    }
  } else if (tid == 0) {
    atomicExch(&g_prefill_status, 1);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)tmem_cols) : "memory");
}

cudaError_t prefill_gemm_dispatch(const void* Wp, const void* SZ, const void* X, void* Y, int T, int N, int K, int log2G,
                                  cudaStream_t st) {
  const int Tpad = (T + 15) / 16 * 16;
  int cols = 32;
  while (cols < Tpad) cols *= 2;
  const size_t smem = 1024 + 2 * ((size_t)kPfRows * 128 + (size_t)Tpad * 128);
  static size_t allowed[kMaxDevices] = {};
  const cudaError_t e = allow_dynamic_smem(prefill_gemm_kernel, smem, allowed);
  if (e != cudaSuccess) return e;
  prefill_gemm_kernel<<<(N + kPfRows - 1) / kPfRows, kPfThreads, smem, st>>>((const uint32_t*)Wp, (const half2*)SZ,
                                                                             (const half*)X, (half*)Y, T, Tpad, N, K,
                                                                             log2G, cols);
  return cudaPeekAtLastError();
}

int prefill_gemm_max_tokens() { return kPfMaxT; }

cudaError_t prefill_gemm_status(int* code) {
  return cudaMemcpyFromSymbol(code, g_prefill_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

}  // namespace b200
