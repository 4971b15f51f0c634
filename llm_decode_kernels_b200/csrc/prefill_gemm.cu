// Batched W4A16 GEMM for the prompt:  Y[T, N] = X[T, K] . dequant(W)[N, K]^T, fp32 accumulation, fp16 out.
//
// The reference processes a prompt token by token through its decode step (runtime/model.py:267-276) and records its
// tensor-core prefill GEMM as cut (RESULTS.md:385-387). With T tokens at once every weight is read once instead of T
// times, and the product is a dense contraction - the one place in this library where the 5th-generation tensor cores
// fit: tcgen05.mma, operands in shared memory, accumulator in tensor memory.
//
// Work unit = one CTA: a 128-row block of W, all T tokens, one contiguous share of K (split s of S). The S CTAs of a
// row block form a thread-block cluster. Per 64-column chunk of K: D[128 features, T tokens] (+)= A[128, 64] .
// B[T, 64]^T as four tcgen05.mma.kind::f16 of K = 16 each.
//   A = the weights. Warps 0-15 read the packed words (8 bytes = 16 weights per thread and chunk, the words of the
//       next eight chunks already in flight) and the groups' (scale, zero), dequantize exactly as dequant_w4a16_kernel does (so
//       the fp16 weights are the format's, bit for bit) and store 16-byte pieces into shared memory in the K-major
//       128-byte-swizzle layout the MMA's descriptor names;
//   B = the activations: one TMA tile copy per chunk (cp.async.bulk.tensor, 128-byte swizzle done by the copy engine,
//       rows past T filled with zeros), issued by warp 17;
//   D = fp32 in tensor memory: 128 lanes (features) x T columns, allocated with tcgen05.alloc; warp 16 issues the MMAs.
// Four to eight shared-memory stages (what fits beside T); tcgen05.commit arrives on a stage's mbarrier when the tensor core has finished with it.
// Epilogue: warps 0-15 read the accumulator with tcgen05.ld and park it as fp32 in shared memory (over the stages,
// which are idle by then); after a cluster barrier CTA r of the cluster sums, for every S-th token, the S partial
// tiles in split order through distributed shared memory, rounds to fp16 and stores whole rows of Y. The sum order
// is fixed, so results do not depend on timing.
// Every wait on an mbarrier is bounded; a wait that runs out raises the CTA's fail flag, the other roles see it in
// their own waits, the CTA waits (bounded) for its copies in flight, still takes part in the cluster barriers, frees
// its tensor memory and returns; b200_gemm_w4a16_status then reports 1.
#include "common.cuh"
#include <cuda.h>

namespace b200 {

namespace {

constexpr int kPfDequantWarps = 16;
constexpr int kPfThreads = (kPfDequantWarps + 2) * 32;   // + one warp for MMA issue + one for TMA issue
constexpr int kPfRows = 128;           // rows of W per CTA = M of the MMA
constexpr int kPfChunk = 64;           // K elements per stage: one 128-byte swizzle row of fp16
constexpr int kPfMinStages = 4, kPfMaxStages = 8;   // shared-memory stages: as many as fit (4 at 256 tokens, 8 up to 64)
constexpr size_t kPfSmemLimit = 231424;            // dynamic shared memory the kernel may ask for (227 KB less its static part)
constexpr int kPfPrefetch = 8;         // chunks of packed words a dequantizing thread holds in registers ahead of use
constexpr int kPfMaxT = 256;           // tokens per call = N of the MMA (multiple of 16)
constexpr int kPfMaxSplit = 8;         // portable cluster size
constexpr int kPfSpinLimit = 1 << 22;
static_assert(1024 + (size_t)kPfMinStages * (kPfRows * 128 + kPfMaxT * 128) <= kPfSmemLimit, "four stages at 256 tokens");

__device__ int g_prefill_status = 0;   // 0, or 1 once a bounded wait inside prefill_gemm_kernel ran out

DEVI uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

DEVI void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(b)), "r"(count));
}
DEVI void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(b)) : "memory");
}
DEVI void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(b)), "r"(bytes) : "memory");
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
// false if the phase did not complete within the limit, or another role of the CTA has given up (fail flag).
// SLEEP_NS > 0: back off between polls. The dequantizing warps run stages ahead and then wait; eighteen warps polling
// at full rate would take the issue slots the one MMA-issuing thread needs.
template <int SLEEP_NS>
DEVI bool mbar_wait_bounded(uint64_t* b, uint32_t parity, volatile int* fail) {
  if (mbar_try_wait(b, parity)) return true;
#pragma unroll 1
  for (int i = 0; i < kPfSpinLimit; ++i) {
    if (SLEEP_NS > 0) __nanosleep(SLEEP_NS);
    if (mbar_try_wait(b, parity)) return true;
    if (fail && (i & 63) == 63 && *fail) return false;
  }
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

// one 2-D tile of the activations into this CTA's shared memory; completion counts bytes on the stage's mbarrier
DEVI void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_addr(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
      : "memory");
}

// byte offset of 16-byte piece c (0..7) of row r inside a swizzled tile
DEVI uint32_t sw128_offset(int r, int c) { return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4)); }

DEVI void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// 16 bytes from the same shared-memory offset in CTA `rank` of the cluster
DEVI float4 ld_cluster_f4(uint32_t local_saddr, uint32_t rank) {
  uint32_t ra;
  float4 v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(local_saddr), "r"(rank));
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(ra)
               : "memory");
  return v;
}

struct PfShared {   // static shared memory of the kernel
  uint64_t a_full[kPfMaxStages], b_full[kPfMaxStages], mma_done[kPfMaxStages], acc_done;
  uint32_t tmem_base;
  int fail;
};

}  // namespace

// xmap: tensor map of X fp16 [T, K] with boxes of 64 columns x Tpad rows, 128-byte swizzle. Wp int32 [N, K/8] and SZ
// half2 [N, K >> log2G] are the quantizer's row-major tensors; Y fp16 [T, N]. Tpad = T rounded up to a multiple of 16
// (the MMA's N); K % 64 == 0; the group size a multiple of 64. Grid (row blocks, S), clusters of (1, S, 1).
__global__ void __launch_bounds__(kPfThreads, 1)
prefill_gemm_kernel(const __grid_constant__ CUtensorMap xmap, const uint32_t* __restrict__ Wp,
                    const half2* __restrict__ SZ, half* __restrict__ Y, int T, int Tpad, int N, int K, int log2G,
                    int tmem_cols, int ns) {
  extern __shared__ uint8_t pf_raw[];
  __shared__ PfShared sh;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~(uintptr_t)1023);
  const int a_bytes = kPfRows * 128, b_bytes = Tpad * 128, stage_bytes = a_bytes + b_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int S = gridDim.y, split = blockIdx.y;   // split == rank of this CTA in its cluster
  const int nchunks = K / kPfChunk, c_begin = split * nchunks / S, n = (split + 1) * nchunks / S - c_begin;
  const int row0 = blockIdx.x * kPfRows;
  volatile int* fail = &sh.fail;
  pdl_launch_dependents();   // the next kernel's prologue may overlap; it waits for this grid's completion itself

  if (warp == 0) {   // one warp allocates the accumulator's columns of tensor memory for the CTA
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&sh.tmem_base)),
                 "r"((uint32_t)tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  if (tid == 0) {
    for (int s = 0; s < ns; ++s) {
      mbar_init(&sh.a_full[s], kPfDequantWarps);
      mbar_init(&sh.b_full[s], 1);
      mbar_init(&sh.mma_done[s], 1);
    }
    mbar_init(&sh.acc_done, 1);
    sh.fail = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem_base;

  if (warp < kPfDequantWarps) {
    // ---- A: thread p dequantizes a quarter row (16 weights) of every chunk: row p / 4, 16-byte pieces 2 (p % 4) ..
    // Many warps with little work each: the dequantization is a chain of dependent half2 operations, and it is the
    // number of warps per scheduler that hides their latency.
    const int r = tid >> 2, qt = tid & 3, row = row0 + r;
    const bool valid = row < N;
    const int words = K >> 3, ng = K >> log2G;
    const uint2* wp = reinterpret_cast<const uint2*>(Wp + (size_t)(valid ? row : 0) * words) + qt;
    const half2* szp = SZ + (size_t)(valid ? row : 0) * ng;
    const half2 k1024 = __float2half2_rn(1024.f);
    // ring of the next kPfPrefetch chunks' words and (scale, zero) in registers: eight loads in flight per thread
    // cover the DRAM latency at one chunk per few hundred cycles
    uint2 rw[kPfPrefetch];
    half2 rsz[kPfPrefetch];
#pragma unroll
    for (int u = 0; u < kPfPrefetch; ++u) {
      rw[u] = make_uint2(0u, 0u);
      rsz[u] = __float2half2_rn(0.f);
      if (valid && u < n) {
        rw[u] = __ldg(wp + 4 * (c_begin + u));
        rsz[u] = __ldg(szp + (((c_begin + u) * kPfChunk + qt * 16) >> log2G));
      }
    }
    bool go = true;
    int s = 0, use = 0;   // stage of chunk j and how often the stage has been used before
    for (int j0 = 0; j0 < n && go; j0 += kPfPrefetch) {
#pragma unroll
      for (int u = 0; u < kPfPrefetch; ++u) {
        const int j = j0 + u;
        if (j >= n) break;
        const uint2 cw = rw[u];
        const half2 csz = rsz[u];
        if (valid && j + kPfPrefetch < n) {
          rw[u] = __ldg(wp + 4 * (c_begin + j + kPfPrefetch));
          rsz[u] = __ldg(szp + (((c_begin + j + kPfPrefetch) * kPfChunk + qt * 16) >> log2G));
        }
        // the decision is the warp's, so that its lanes stay together for the __syncwarp below
        if (use >= 1 && !__all_sync(0xffffffffu, mbar_wait_bounded<128>(&sh.mma_done[s], (use - 1) & 1, fail))) {
          *fail = 1;
          go = false;
          break;
        }
        // (q - z) * s per pair of weights, the arithmetic of dequant_w4a16_kernel. The nibbles at bits 4-7 / 20-23 are
        // taken where they stand, as 1024 + 16 q, and multiplied by s / 16 - the same real product, hence the same
        // rounding, whenever s / 16 is exact in fp16 (checked; a subnormal scale takes the shifted form). That leaves
        // one shift and four logic operations per word on the ALU pipe, which is what bounds this loop.
        const half sc = __low2half(csz), sc16 = __hmul(sc, __float2half_rn(0.0625f));
        const half2 s2 = __half2half2(sc), s2h = __half2half2(sc16);
        const half2 zl = __hadd2(__half2half2(__high2half(csz)), k1024);
        const half2 zh = __hfma2(__half2half2(__high2half(csz)), __float2half2_rn(16.f), k1024);
        // ... and 1024 + 16 z must be sixteen times what 1024 + z rounds z to (it is, for the format's integer zeros)
        const bool exact16 = __heq(__hmul(sc16, __float2half_rn(16.f)), sc) &&
                             __heq(__hsub(__low2half(zh), __low2half(k1024)),
                                   __hmul(__hsub(__low2half(zl), __low2half(k1024)), __float2half_rn(16.f)));
        const uint32_t w2[2] = {cw.x, cw.y};
        uint8_t* dst = base + s * stage_bytes;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint32_t w = w2[q], w8 = w >> 8;
          uint4 o;
          o.x = as_u32(__hmul2(__hsub2(nib_lo(w), zl), s2));
          o.z = as_u32(__hmul2(__hsub2(nib_lo(w8), zl), s2));
          if (exact16) {
            o.y = as_u32(__hmul2(__hsub2(as_h2((w & 0x00F000F0u) | 0x64006400u), zh), s2h));
            o.w = as_u32(__hmul2(__hsub2(as_h2((w8 & 0x00F000F0u) | 0x64006400u), zh), s2h));
          } else {
            o.y = as_u32(__hmul2(__hsub2(nib_lo(w >> 4), zl), s2));
            o.w = as_u32(__hmul2(__hsub2(nib_lo(w >> 12), zl), s2));
          }
          // rows past N carry zero words and a zero scale: their products are zeros without a special case
          *reinterpret_cast<uint4*>(dst + sw128_offset(r, 2 * qt + q)) = o;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy stores -> visible to the tensor core
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.a_full[s]);   // one arrival per warp: arrivals on one mbarrier serialize
        if (++s == ns) s = 0, ++use;
      }
    }
  } else if (warp == kPfDequantWarps) {
    // ---- MMA issue: one thread
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(kPfRows, Tpad);
      bool ok = true;
      for (int j = 0, s = 0, use = 0; j < n && ok; ++j) {
        ok = mbar_wait_bounded<0>(&sh.a_full[s], use & 1, fail) && mbar_wait_bounded<0>(&sh.b_full[s], use & 1, fail);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = umma_desc_sw128(smem_addr(base + s * stage_bytes));
        const uint64_t db = umma_desc_sw128(smem_addr(base + s * stage_bytes + a_bytes));
#pragma unroll
        for (int k = 0; k < kPfChunk / 16; ++k)   // 16 fp16 = 32 bytes further along the swizzled row: +2 in units of 16 B
          umma_f16(tmem, da + 2 * k, db + 2 * k, idesc, (j | k) != 0 ? 1u : 0u);
        umma_commit(&sh.mma_done[s]);
        if (++s == ns) s = 0, ++use;
      }
      if (ok) umma_commit(&sh.acc_done);   // arrives when every MMA of this CTA has completed
      else *fail = 1;
    }
  } else {
    // ---- B: one thread issues the tile copies of X
    if (lane == 0) {
      pdl_wait();   // X is the predecessor's output; the weights, read by the other warps meanwhile, are not
      int issued = 0;
      for (int j = 0, s = 0, use = 0; j < n; ++j) {
        if (use >= 1 && !mbar_wait_bounded<32>(&sh.mma_done[s], (use - 1) & 1, fail)) {
          *fail = 1;
          break;
        }
        mbar_expect_tx(&sh.b_full[s], (uint32_t)b_bytes);
        tma_load_2d(base + s * stage_bytes + a_bytes, &xmap, (c_begin + j) * kPfChunk, 0, &sh.b_full[s]);
        issued = j + 1;
        if (++s == ns) s = 0, ++use;
      }
      if (*fail)   // giving up: let the copies still in flight land before the CTA's shared memory goes away
        for (int j = issued > ns ? issued - ns : 0; j < issued; ++j)
          mbar_wait_bounded<64>(&sh.b_full[j % ns], (j / ns) & 1, nullptr);
    }
  }
  __syncwarp();

  // ---- epilogue 1: accumulator -> fp32 partial tile P[token][128 features] in shared memory (over the idle stages)
  float* P = reinterpret_cast<float*>(base);
  if (warp < kPfDequantWarps) {
    const bool ok = mbar_wait_bounded<256>(&sh.acc_done, 0, fail);
    if (!ok) *fail = 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (ok) {
      // a warp reaches the 32 lanes 32 (warp % 4) ..; the four warps that share them take turns over the column groups
      const int q = warp & 3;
      for (int c0 = 16 * (warp >> 2); c0 < Tpad; c0 += 16 * (kPfDequantWarps / 4)) {
        uint32_t v[16];
        const uint32_t taddr = tmem + ((uint32_t)(32 * q) << 16) + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) P[(c0 + j) * kPfRows + 32 * q + lane] = __uint_as_float(v[j]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync_all();   // every CTA of the row block has parked its partial tile

  // ---- epilogue 2: CTA `split` finishes tokens split, split + S, ...: sum over the cluster in split order, store rows
  pdl_wait();   // Y may still be read by the kernel before this one
  if (warp < kPfDequantWarps) {
    const int g4 = (tid & 31) * 4, feature = row0 + g4;
    const bool vec = (N & 3) == 0 && (reinterpret_cast<uintptr_t>(Y) & 7) == 0;
    for (int t = warp * S + split; t < T; t += kPfDequantWarps * S) {
      const uint32_t local = smem_addr(P + t * kPfRows + g4);
      float4 v[kPfMaxSplit];   // all remote reads in flight at once, then the sum in split order
#pragma unroll
      for (int s = 0; s < kPfMaxSplit; ++s)
        if (s < S) v[s] = ld_cluster_f4(local, (uint32_t)s);
      float4 acc = v[0];
#pragma unroll
      for (int s = 1; s < kPfMaxSplit; ++s)
        if (s < S) acc.x += v[s].x, acc.y += v[s].y, acc.z += v[s].z, acc.w += v[s].w;
      half* y = Y + (size_t)t * N + feature;
      if (vec && feature + 3 < N) {
        uint2 o;
        o.x = as_u32(__floats2half2_rn(acc.x, acc.y));
        o.y = as_u32(__floats2half2_rn(acc.z, acc.w));
        *reinterpret_cast<uint2*>(y) = o;
      } else {
        const float a4[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (feature + e < N) y[e] = __float2half(a4[e]);
      }
    }
  }
  cluster_sync_all();   // nobody's shared memory goes away while a peer still reads it
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)tmem_cols) : "memory");
  if (tid == 0 && *fail) atomicExch(&g_prefill_status, 1);
}

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query: the library does not link libcuda
EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

}  // namespace

// How many ways K is split for a matrix of N rows: the largest power of two, up to the portable cluster size, for
// which every cluster of the grid is resident at once (the occupancy query knows how many clusters of that size the
// GPU's processor groups hold) and every split keeps at least two chunks.
static void cluster_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int blocks, int S, size_t smem,
                           cudaStream_t st) {   // attr: array of two
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(blocks, S, 1);
  cfg->blockDim = dim3(kPfThreads, 1, 1);
  cfg->dynamicSmemBytes = smem;
  cfg->stream = st;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 2;
}

static int max_resident_clusters(int S, size_t smem) {   // per device and cluster size, asked once
  static int known[kMaxDevices][kPfMaxSplit + 1] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 0;
  if (known[dev][S] == 0) {
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    cluster_config(&cfg, attr, 1, S, smem, nullptr);
    int num = 0;
    if (cudaOccupancyMaxActiveClusters(&num, prefill_gemm_kernel, &cfg) != cudaSuccess) {
      (void)cudaGetLastError();
      num = 0;
    }
    known[dev][S] = num > 0 ? num : -1;
  }
  return known[dev][S] > 0 ? known[dev][S] : 0;
}

int prefill_gemm_splits(int N, int K, size_t smem) {
  const int blocks = (N + kPfRows - 1) / kPfRows, nchunks = K / kPfChunk;
  for (int S = kPfMaxSplit; S > 1; S /= 2)
    if (nchunks / S >= 2 && blocks <= max_resident_clusters(S, smem)) return S;
  return 1;
}

cudaError_t prefill_gemm_dispatch(const void* Wp, const void* SZ, const void* X, void* Y, int T, int N, int K, int log2G,
                                  cudaStream_t st) {
  const int Tpad = (T + 15) / 16 * 16;
  int cols = 32;
  while (cols < Tpad) cols *= 2;
  const EncodeTiledFn encode = encode_tiled();
  if (!encode) return cudaErrorNotSupported;
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)T}, strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kPfChunk, (cuuint32_t)Tpad}, estr[2] = {1, 1};
  if (encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(X), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return cudaErrorInvalidValue;
  const size_t stage = (size_t)kPfRows * 128 + (size_t)Tpad * 128;
  int ns = (int)((kPfSmemLimit - 1024) / stage);
  ns = ns > kPfMaxStages ? kPfMaxStages : ns;   // >= kPfMinStages: four stages of the largest tile fit
  const size_t smem = 1024 + ns * stage;
  // the kernel is allowed, and its cluster occupancy asked, at the largest tile (T = 256): one CTA per SM at every T
  const size_t smem_max = kPfSmemLimit;
  static size_t allowed[kMaxDevices] = {};
  const cudaError_t e = allow_dynamic_smem(prefill_gemm_kernel, smem_max, allowed);
  if (e != cudaSuccess) return e;
  const int S = prefill_gemm_splits(N, K, smem_max);
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[2];
  cluster_config(&cfg, attr, (N + kPfRows - 1) / kPfRows, S, smem, st);
  return cudaLaunchKernelEx(&cfg, prefill_gemm_kernel, xmap, (const uint32_t*)Wp, (const half2*)SZ, (half*)Y, T, Tpad, N,
                            K, log2G, cols, ns);
}

int prefill_gemm_max_tokens() { return kPfMaxT; }

cudaError_t prefill_gemm_status(int* code) {
  return cudaMemcpyFromSymbol(code, g_prefill_status, sizeof(int), 0, cudaMemcpyDeviceToHost);
}

}  // namespace b200
