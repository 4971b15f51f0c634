// Paged split-K decode attention (one query token per sequence, grouped-query heads) and its combine step.
//
// Replaces paged_attention_launch of the reference (kernels/paged_attention.cu:429-461, bound at
// kernels/bindings.cpp:45-62), generalised to a batch of sequences and to head_dim 64 or 128.
//
// Layout: caches [pages, n_kv, P, D] fp16 (P = 2^log2P tokens per page); block table bt[b, i] = physical page
// of tokens [i P, (i+1) P) of sequence b; context length of sequence b = pos[b] + 1, read on the device so one
// captured graph serves every step. Split s of a sequence owns tokens [s PS, min(ctx, (s+1) PS)).
//
// Three partial kernels (the `version` of the entry points) share the grid (n_kv, max_splits, B); a block handles ALL
// heads of one kv group, so every K/V byte is fetched from HBM once. Version 3, paged_attn_mma_kernel, is the default
// and is described where it is defined; it builds on version 2:
//
// paged_attn_staged_kernel (version 2; like version 3 for pages of 8..64 tokens and splits that start on a page boundary):
// the split's K and V pages are pulled into a shared-memory ring by bulk async copies (cp.async.bulk + mbarrier
// transaction counts), one copy per page, issued by the lanes of warp 0 several 64-token tiles ahead of the
// arithmetic. A decode-attention block has little to compute and a lot to fetch; with register loads the bytes in
// flight per SM are limited by what a few warps can hold in registers (the first kernel of this file moved 0.4-1.1
// TB/s), while the ring keeps 64-190 KB per SM in flight. Arithmetic out of the ring, per warp and 16 tokens:
//   scores : D/8 lanes share a token, each holds 8 dims of every head's query in registers, multiplies its 16-byte
//            piece of the K row into HPG partial sums, and a folding butterfly (half of the values travel at every
//            step) leaves lane (token, head) with the finished score: D/8 - 1 + log2 shuffles instead of HPG * log2;
//   softmax: per-warp running max / sum per head, probabilities and the rescale factor go through a small
//            per-warp shared tile;
//   output : lane l owns D/32 output dims of every head; per token one V read, the token's HPG probabilities
//            (broadcast), HPG * D/32 FMAs.
//
// paged_attn_partial_kernel (any page size, any split size): each warp walks its own 32-token tiles with a private
// online-softmax state (no block barrier in the loop), K/V by register loads:
//   scores : lane t owns token t of the tile, holds that K row in registers and dots it with every head's
//            query (pre-scaled by 1/sqrt(D), fp32, broadcast reads from shared memory) - no shuffles;
//   p      : exp(score - running max) goes to a per-warp shared tile [32 tokens][HPG heads];
//   output : lane l owns D/32 consecutive output dims of every head and walks the tile's V rows
//            (each row one coalesced 128- or 256-byte read), acc[h][d] += p[t][h] * v[t][d].
// The four warps are merged once through shared memory with the max-rescale rule; a block that is the
// only live split of its sequence normalises and writes fp16 `out` itself, otherwise it writes
// un-normalised fp32 partials (o, m, l) and the combine kernel finishes:
//   M = max_s m_s,  L = sum_s l_s e^(m_s - M),  O = sum_s o_s e^(m_s - M) / L.
#include "common.cuh"
#include <math_constants.h>

namespace b200 {

constexpr int kAttnThreads = 128;
constexpr int kAttnWarps = kAttnThreads / 32;

template <int D, int HPG>
__global__ void __launch_bounds__(kAttnThreads)
paged_attn_partial_kernel(const half* __restrict__ q, const half* __restrict__ kc, const half* __restrict__ vc,
                          const int* __restrict__ bt, int bt_stride, const int* __restrict__ pos_ptr, int n_kv,
                          int log2P, int PS, float scale, float* __restrict__ o_part, float* __restrict__ m_part,
                          float* __restrict__ l_part, half* __restrict__ out, int max_splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DPL = D / 32;      // output dims owned by one lane
  constexpr int CHUNKS = D / 8;    // 16-byte chunks per K/V row
  __shared__ __align__(16) float q_s[HPG][D];
  __shared__ __align__(16) float p_s[kAttnWarps][32][HPG];
  __shared__ long long row_s[kAttnWarps][32];  // element offset of each tile token's row in the caches
  __shared__ float wm[kAttnWarps][HPG], wl[kAttnWarps][HPG];
  __shared__ float wo[kAttnWarps][HPG][D];

  const int kvh = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int n_q = n_kv * HPG;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (split >= nsplit) return;
  const int t0 = split * PS, t1 = min(ctx, t0 + PS);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* btb = bt + (size_t)b * bt_stride;
  const int pmask = (1 << log2P) - 1;

  for (int i = tid; i < HPG * D; i += kAttnThreads)
    q_s[i / D][i % D] = __half2float(q[((size_t)b * n_q + kvh * HPG) * D + i]) * scale;
  __syncthreads();

  float m[HPG], l[HPG], acc[HPG][DPL];
#pragma unroll
  for (int h = 0; h < HPG; ++h) {
    m[h] = -CUDART_INF_F;
    l[h] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;
  }

  for (int tile = t0 + 32 * warp; tile < t1; tile += 32 * kAttnWarps) {
    const int t = tile + lane;
    const bool valid = t < t1;
    const int tc = valid ? t : t1 - 1;
    const long long row = ((((long long)btb[tc >> log2P] * n_kv + kvh) << log2P) + (tc & pmask)) * D;
    row_s[warp][lane] = row;

    // ---- scores: this lane's token against every head of the group
    float s[HPG];
#pragma unroll
    for (int h = 0; h < HPG; ++h) s[h] = 0.f;
    const uint4* kp = reinterpret_cast<const uint4*>(kc + row);
#pragma unroll
    for (int c0 = 0; c0 < CHUNKS; c0 += 8) {
      uint4 kv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) kv[c] = __ldg(kp + c0 + c);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float kf[8];
        unpack8(kv[c], kf);
#pragma unroll
        for (int h = 0; h < HPG; ++h) {
          const float4 qa = *reinterpret_cast<const float4*>(&q_s[h][(c0 + c) * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&q_s[h][(c0 + c) * 8 + 4]);
          s[h] = fmaf(kf[0], qa.x, fmaf(kf[1], qa.y, fmaf(kf[2], qa.z, fmaf(kf[3], qa.w, s[h]))));
          s[h] = fmaf(kf[4], qb.x, fmaf(kf[5], qb.y, fmaf(kf[6], qb.z, fmaf(kf[7], qb.w, s[h]))));
        }
      }
    }

    // ---- online softmax update (m uniform across the warp, l kept as per-lane partial sums)
#pragma unroll
    for (int h = 0; h < HPG; ++h) {
      const float sv = valid ? s[h] : -CUDART_INF_F;
      const float mn = fmaxf(m[h], warp_max(sv));
      const float alpha = __expf(m[h] - mn);  // first tile: e^(-inf) = 0
      const float p = __expf(sv - mn);        // masked lane: 0
      l[h] = l[h] * alpha + p;
      m[h] = mn;
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[h][d] *= alpha;
      p_s[warp][lane][h] = p;
    }
    __syncwarp();

    // ---- output: walk the tile's V rows, 4 rows in flight
    const int nt = min(32, t1 - tile);
    for (int j0 = 0; j0 < nt; j0 += 4) {
      float vf[4][DPL];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int jj = min(j0 + j, nt - 1);
        const half* vp = vc + row_s[warp][jj] + lane * DPL;
        if (DPL == 2) {
          const float2 f = __half22float2(*reinterpret_cast<const half2*>(vp));
          vf[j][0] = f.x; vf[j][1] = f.y;
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(vp);
          const float2 f0 = __half22float2(as_h2(u.x)), f1 = __half22float2(as_h2(u.y));
          vf[j][0] = f0.x; vf[j][1] = f0.y; vf[j][DPL - 2] = f1.x; vf[j][DPL - 1] = f1.y;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (j0 + j < nt) {
#pragma unroll
          for (int h0 = 0; h0 < HPG; h0 += 4) {
            float ph[4];
            if (HPG >= 4) {
              const float4 p4 = *reinterpret_cast<const float4*>(&p_s[warp][j0 + j][h0]);
              ph[0] = p4.x; ph[1] = p4.y; ph[2] = p4.z; ph[3] = p4.w;
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) ph[k] = k < HPG ? p_s[warp][j0 + j][k < HPG ? k : 0] : 0.f;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              if (h0 + k < HPG) {
#pragma unroll
                for (int d = 0; d < DPL; ++d) acc[h0 + k][d] = fmaf(ph[k], vf[j][d], acc[h0 + k][d]);
              }
            }
          }
        }
      }
    }
    __syncwarp();  // p_s / row_s are rewritten by the next tile
  }

  // ---- merge the warps
#pragma unroll
  for (int h = 0; h < HPG; ++h) {
    const float lw = warp_sum(l[h]);
    if (lane == 0) { wm[warp][h] = m[h]; wl[warp][h] = lw; }
#pragma unroll
    for (int d = 0; d < DPL; ++d) wo[warp][h][lane * DPL + d] = acc[h][d];
  }
  __syncthreads();
  for (int i = tid; i < HPG * D; i += kAttnThreads) {
    const int h = i / D, d = i % D, head = kvh * HPG + h;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, wm[w][h]);
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float a = __expf(wm[w][h] - M);  // a warp that had no tile: e^(-inf) = 0
      o = fmaf(a, wo[w][h][d], o);
      L = fmaf(a, wl[w][h], L);
    }
    const size_t hq = (size_t)b * n_q + head;
    if (nsplit == 1) {
      out[hq * D + d] = __float2half(o / L);
    } else {
      o_part[(hq * max_splits + split) * D + d] = o;
      if (d == 0) { m_part[hq * max_splits + split] = M; l_part[hq * max_splits + split] = L; }
    }
  }
}

// ---- staged kernel ---------------------------------------------------------------------------------------------------
namespace {

__device__ int g_attn_status = 0;   // set to 1 by a block whose bounded wait for its own copies ran out

constexpr int kStageTokens = 64;
constexpr int kWaitLimit = 1 << 20;

DEVI uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI bool bar_wait(uint64_t* bar, uint32_t parity, int limit) {
  for (int i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(sm_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// v[0..N) are per-lane partial sums of N heads; lanes that differ in the bits below 2*OFF hold pieces of the same
// token. Every step sends half of the values to the partner lane and keeps the other half, so after log2(N) steps a
// lane holds one head's sum over those lanes; remaining steps (more lanes than heads) are plain sums. The lane's
// head is ((lane mod lanes-per-token) * HPG) / lanes-per-token.
template <int N, int OFF>
DEVI float fold_heads(float* v, int lane) {
  if constexpr (N > 1) {
    const bool up = lane & OFF;
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
      const float keep = up ? v[i + N / 2] : v[i];
      const float send = up ? v[i] : v[i + N / 2];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, OFF);
    }
    return fold_heads<N / 2, OFF / 2>(v, lane);
  } else if constexpr (OFF >= 1) {
    v[0] += __shfl_xor_sync(0xffffffffu, v[0], OFF);
    return fold_heads<1, OFF / 2>(v, lane);
  } else {
    return v[0];
  }
}

// D (16x8, fp32) += A (16x16, fp16, row) * B (16x8, fp16, col)
DEVI void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace

template <int D>
constexpr int attn_ring_stages() { return 3; }   // 48 KB (head_dim 64: four blocks per SM) or 96 KB (128: two)
template <int D>
constexpr size_t attn_ring_bytes() { return (size_t)attn_ring_stages<D>() * 2 * kStageTokens * D * sizeof(half); }

template <int D, int HPG>
__global__ void __launch_bounds__(kAttnThreads, D == 64 ? 3 : 2)
paged_attn_staged_kernel(const half* __restrict__ q, const half* __restrict__ kc, const half* __restrict__ vc,
                         const int* __restrict__ bt, int bt_stride, const int* __restrict__ pos_ptr, int n_kv,
                         int log2P, int PS, float scale, float* __restrict__ o_part, float* __restrict__ m_part,
                         float* __restrict__ l_part, half* __restrict__ out, int max_splits) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int T = kStageTokens;
  constexpr int NS = attn_ring_stages<D>();
  constexpr int LPT = D / 8;               // lanes that share one token in the score phase
  constexpr int TPP = 32 / LPT;            // tokens per pass of a warp
  constexpr int TW = T / kAttnWarps;       // tokens of a tile owned by one warp
  constexpr int NP = TW / TPP;             // passes per tile
  constexpr int DPL = D / 32;              // output dims owned by one lane
  constexpr int DUP = LPT / HPG;           // lanes that end up with the same (token, head) score
  constexpr int STAGE_ELEMS = 2 * T * D;   // K tile then V tile
  extern __shared__ __align__(128) uint8_t ring_raw[];
  half* ring = reinterpret_cast<half*>(ring_raw);
  __shared__ uint64_t full[NS];
  __shared__ __align__(16) float q_s[HPG][D];
  __shared__ __align__(16) float p_s[kAttnWarps][TW][HPG];
  __shared__ __align__(16) float a_s[kAttnWarps][8];
  __shared__ float wm[kAttnWarps][HPG], wl[kAttnWarps][HPG];

  const int kvh = blockIdx.x, split = blockIdx.y, b = blockIdx.z;
  const int n_q = n_kv * HPG;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (split >= nsplit) return;
  const int t0 = split * PS, t1 = min(ctx, t0 + PS);
  const int ntiles = (t1 - t0 + T - 1) / T;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* btb = bt + (size_t)b * bt_stride;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < NS; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm_u32(&full[i])));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < HPG * D; i += kAttnThreads)
    q_s[i / D][i % D] = __half2float(q[((size_t)b * n_q + kvh * HPG) * D + i]) * scale;
  __syncthreads();

  // warp 0: one bulk copy per K page and per V page of tile i (lane = page), all landing on the tile's barrier
  const uint32_t page_bytes = (uint32_t)(D * sizeof(half)) << log2P;
  auto issue = [&](int i) {
    const int slot = i % NS, tok0 = t0 + i * T;
    const int npg = min(T >> log2P, (t1 - tok0 + (1 << log2P) - 1) >> log2P);
    if (lane == 0)
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sm_u32(&full[slot])),
                   "r"(2u * npg * page_bytes)
                   : "memory");
    __syncwarp();
    if (lane < 2 * npg) {
      const int isv = lane >= npg, pg = lane - isv * npg;
      const size_t off = (((size_t)__ldg(btb + (tok0 >> log2P) + pg) * n_kv + kvh) << log2P) * D;
      const half* src = (isv ? vc : kc) + off;
      half* dst = ring + (size_t)slot * STAGE_ELEMS + (isv ? T * D : 0) + ((size_t)pg << log2P) * D;
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                       sm_u32(dst)),
                   "l"(src), "r"(page_bytes), "r"(sm_u32(&full[slot]))
                   : "memory");
    }
  };
  if (warp == 0)
    for (int i = 0; i < min(NS, ntiles); ++i) issue(i);

  const int ch = lane & (LPT - 1), tsub = lane / LPT;
  const int head = ch / DUP;
  const bool writer = (ch & (DUP - 1)) == 0;   // one lane per (token, head)
  float qr[HPG][8];
#pragma unroll
  for (int h = 0; h < HPG; ++h) {
    const float4 a = *reinterpret_cast<const float4*>(&q_s[h][ch * 8]);
    const float4 c = *reinterpret_cast<const float4*>(&q_s[h][ch * 8 + 4]);
    qr[h][0] = a.x; qr[h][1] = a.y; qr[h][2] = a.z; qr[h][3] = a.w;
    qr[h][4] = c.x; qr[h][5] = c.y; qr[h][6] = c.z; qr[h][7] = c.w;
  }
  float m = -CUDART_INF_F, l = 0.f, acc[HPG][DPL];
#pragma unroll
  for (int h = 0; h < HPG; ++h)
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[h][d] = 0.f;

  int failed_at = -1;
  for (int i = 0; i < ntiles; ++i) {
    const int slot = i % NS;
    const bool ok = bar_wait(&full[slot], (uint32_t)(i / NS) & 1u, kWaitLimit);
    const half* kt = ring + (size_t)slot * STAGE_ELEMS;
    const half* vt = kt + T * D;
    const int nt = min(T, t1 - t0 - i * T);
    const int tok0 = warp * TW;
    if (ok && tok0 < nt) {
      float s[NP];
#pragma unroll
      for (int ps = 0; ps < NP; ++ps) {
        const int j = tok0 + ps * TPP + tsub;   // rows at or beyond nt hold stale bytes: computed, then masked
        float kf[8], part[HPG];
        unpack8(*reinterpret_cast<const uint4*>(kt + (size_t)j * D + ch * 8), kf);
#pragma unroll
        for (int h = 0; h < HPG; ++h) part[h] = kf[0] * qr[h][0];
#pragma unroll
        for (int d = 1; d < 8; ++d)
#pragma unroll
          for (int h = 0; h < HPG; ++h) part[h] = fmaf(kf[d], qr[h][d], part[h]);
        const float sv = fold_heads<HPG, LPT / 2>(part, lane);
        s[ps] = j < nt ? sv : -CUDART_INF_F;
      }
      float mx = s[0];
#pragma unroll
      for (int ps = 1; ps < NP; ++ps) mx = fmaxf(mx, s[ps]);
#pragma unroll
      for (int o = LPT; o < 32; o <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m, mx);            // finite: the warp's first token of the tile is valid
      const float alpha = __expf(m - mn);       // first tile: e^(-inf) = 0
      m = mn;
      float lsum = 0.f;
#pragma unroll
      for (int ps = 0; ps < NP; ++ps) {
        const float p = __expf(s[ps] - mn);     // masked token: 0
        lsum += p;
        if (writer) p_s[warp][ps * TPP + tsub][head] = p;
      }
      l = l * alpha + lsum;
      if (writer && tsub == 0) a_s[warp][head] = alpha;
      __syncwarp();
#pragma unroll
      for (int h = 0; h < HPG; ++h) {
        const float al = a_s[warp][h];
#pragma unroll
        for (int d = 0; d < DPL; ++d) acc[h][d] *= al;
      }
      const int nv = min(TW, nt - tok0);        // only valid rows: a stale V row may hold anything, even NaN
#pragma unroll 4
      for (int j = 0; j < nv; ++j) {
        const half* vp = vt + (size_t)(tok0 + j) * D + lane * DPL;
        float vf[DPL];
        if (DPL == 2) {
          const float2 f = __half22float2(*reinterpret_cast<const half2*>(vp));
          vf[0] = f.x; vf[1] = f.y;
        } else {
          const uint2 u = *reinterpret_cast<const uint2*>(vp);
          const float2 f0 = __half22float2(as_h2(u.x)), f1 = __half22float2(as_h2(u.y));
          vf[0] = f0.x; vf[1] = f0.y; vf[DPL - 2] = f1.x; vf[DPL - 1] = f1.y;
        }
        float ph[HPG];
        if (HPG >= 4) {
#pragma unroll
          for (int h0 = 0; h0 < HPG; h0 += 4) {
            const float4 p4 = *reinterpret_cast<const float4*>(&p_s[warp][j][h0]);
            ph[h0] = p4.x; ph[h0 + 1] = p4.y; ph[h0 + 2] = p4.z; ph[h0 + 3] = p4.w;
          }
        } else {
#pragma unroll
          for (int h = 0; h < HPG; ++h) ph[h] = p_s[warp][j][h];
        }
#pragma unroll
        for (int h = 0; h < HPG; ++h)
#pragma unroll
          for (int d = 0; d < DPL; ++d) acc[h][d] = fmaf(ph[h], vf[d], acc[h][d]);
      }
    }
    // every warp is done with the slot (and every thread learns of a wait that ran out) before it is refilled
    if (__syncthreads_or(!ok)) { failed_at = i; break; }
    if (warp == 0 && i + NS < ntiles) issue(i + NS);
  }
  if (failed_at >= 0) {
    // leave only after the copies still in flight have landed (bounded again), and say so
    if (tid == 0) {
      atomicExch(&g_attn_status, 1);
      for (int k = failed_at; k < min(ntiles, failed_at + NS); ++k) bar_wait(&full[k % NS], (uint32_t)(k / NS) & 1u, kWaitLimit);
    }
    __syncthreads();
    return;
  }

  // ---- merge the warps (the ring is free now: reuse it for the per-warp outputs)
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
  if (writer && tsub == 0) { wm[warp][head] = m; wl[warp][head] = l; }
  // every lane needs the running max of every head to publish acc consistently: acc was scaled by the same
  // per-head factors in all lanes, so it is already relative to wm[warp][h]
  float* wo = reinterpret_cast<float*>(ring_raw);   // [kAttnWarps][HPG][D]
#pragma unroll
  for (int h = 0; h < HPG; ++h)
#pragma unroll
    for (int d = 0; d < DPL; ++d) wo[((size_t)warp * HPG + h) * D + lane * DPL + d] = acc[h][d];
  __syncthreads();
  for (int i = tid; i < HPG * D; i += kAttnThreads) {
    const int h = i / D, d = i % D, hd = kvh * HPG + h;
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, wm[w][h]);
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kAttnWarps; ++w) {
      const float a = __expf(wm[w][h] - M);   // a warp that had no token: e^(-inf) = 0
      o = fmaf(a, wo[((size_t)w * HPG + h) * D + d], o);
      L = fmaf(a, wl[w][h], L);
    }
    const size_t hq = (size_t)b * n_q + hd;
    if (nsplit == 1) {
      out[hq * D + d] = __float2half(o / L);
    } else {
      o_part[(hq * max_splits + split) * D + d] = o;
      if (d == 0) { m_part[hq * max_splits + split] = M; l_part[hq * max_splits + split] = L; }
    }
  }
}

// ---- staged kernel, contractions on the tensor cores -----------------------------------------------------------------------
// Same ring, same split / merge protocol as paged_attn_staged_kernel; the two contractions of a tile run as
// mma.sync m16n8k16 (fp16 operands, fp32 accumulators) with the heads of the group as the 16 rows (rows beyond HPG are
// zero). Why tensor cores here and not in the GEMV: with 8 query heads per KV head every K/V byte takes part in 8
// multiply-adds, 16 FLOP per byte of cache; at HBM speed that is more than the fp32 pipes of the chip deliver, and
// paged_attn_staged_kernel is bound by instruction issue at a quarter of the memory bandwidth. The warp-level MMA is
// the right size for it (16 x 8 tiles; the 5th-generation MMA starts at 64 rows and would multiply zeros).
//
// The cache pages arrive by bulk copy, row-major and unpadded, so the textbook fragment loads would meet 8-way bank
// conflicts. Instead both contractions use the freedom to permute the contraction index and the output columns:
//   scores S = Q K^T: lane (g = lane / 4, t = lane % 4) supplies column g of B, i.e. K row "token g" - it reads the
//     D/4 consecutive dims [t D/4, (t+1) D/4) of that row with 16-byte loads and deals them out over the k-steps;
//     Q's fragments are loaded once with the same dealing, so every k-slot pairs the same dim on both sides;
//   output O = P V: the C fragment of S (row g, columns 2t, 2t+1) is exactly the A fragment of P; for B, lane (g, t)
//     reads the 16-byte piece [8g, 8g+8) of its four tokens' V rows and two byte-permutes per register pair
//     transpose token pairs into k-pairs; output column g of n-block j is dim 8g + j.
//
// Copy size. An SM's copy engine handles 15-20 bulk copies per microsecond whatever their size (b200_bw_read_bulk:
// 2 KB copies cap the chip at 3.6-4.5 TB/s with four blocks per SM, 8 KB copies reach 7 TB/s), and one kv head's
// share of a 16-token page is 2 KB. The cache keeps the kv heads of a page next to each other
// ([page][head][slot][dim]), so the kernel is written for KH adjacent kv heads per block (grid.x = n_kv / KH): a
// stage is 64 / KH tokens of KH heads, copied KH heads at a time, and arithmetic warp w works on kv head w % KH.
constexpr int kMmaThreads = kAttnThreads + 32;   // four arithmetic warps + one warp that only issues copies
constexpr int kBtCache = 1024;                   // block-table entries of a split kept in shared memory

//
// ROPE = true folds the step's RoPE + KV-append (rope_append_kernel) into this kernel: `q` is then the raw qkv vector
// of the step ([B, (n_q + 2 n_kv) D], nothing rotated yet). Every block rotates its own query heads while it builds the
// Q fragments. The new token (position pos = ctx - 1) is not in the cache yet: the warp that owns its 16-token block
// in the last split rotates k, patches the K and V rows of the stage in shared memory once the page copy has landed,
// and stores the same rows to the cache in global memory for the steps to come. One launch less per layer.
struct RopeArgs {
  const float *cos_t, *sin_t;   // [max_pos, D/2]
  half *kc_w, *vc_w;            // the caches, writable
};

template <int D, int HPG, int KH, bool ROPE>
__global__ void __launch_bounds__(kMmaThreads, D == 64 ? 4 : 2)
paged_attn_mma_kernel(const half* __restrict__ q, const half* __restrict__ kc, const half* __restrict__ vc,
                      const int* __restrict__ bt, int bt_stride, const int* __restrict__ pos_ptr, int n_kv, int log2P,
                      int PS, float scale, float* __restrict__ o_part, float* __restrict__ m_part,
                      float* __restrict__ l_part, half* __restrict__ out, int max_splits, const RopeArgs ra,
                      int* __restrict__ arrive) {
  static_assert(!ROPE || KH == 1, "the fused RoPE path is written for one kv head per block");
  pdl_launch_dependents();
  pdl_wait();
  constexpr int TS = kStageTokens / KH;    // tokens per ring stage (of each of the KH heads)
  constexpr int NS = attn_ring_stages<D>();
  constexpr int WPH = kAttnWarps / KH;     // arithmetic warps per kv head, 16 tokens of a stage each
  constexpr int KS = D / 16;               // k-steps of the score contraction
  constexpr int CH = D / 32;               // 16-byte pieces of a K row per lane
  constexpr int VC = D / 64;               // 16-byte pieces of a V row per lane
  constexpr int NB = D / 8;                // n-blocks of the output
  constexpr int HALF_STAGE = kStageTokens * D;   // K part of a stage, then the V part
  static_assert(TS == 16 * WPH, "one warp owns 16 tokens of a stage");
  extern __shared__ __align__(128) uint8_t ring_raw[];
  half* ring = reinterpret_cast<half*>(ring_raw);
  __shared__ uint64_t full[NS], empty[NS];
  __shared__ float wm[kAttnWarps][8], wl[kAttnWarps][8];
  __shared__ int bt_s[kBtCache];
  __shared__ int fail_s, last_s;

  const int kvh0 = blockIdx.x * KH, split = blockIdx.y, b = blockIdx.z;
  const int n_q = n_kv * HPG;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (split >= nsplit) return;
  const int t0 = split * PS, t1 = min(ctx, t0 + PS);
  const int ntiles = (t1 - t0 + TS - 1) / TS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  const int* btb = bt + (size_t)b * bt_stride;
  const int pmask = (1 << log2P) - 1;

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < NS; ++i) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(sm_u32(&full[i])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(sm_u32(&empty[i])), "n"(kAttnWarps));
    }
    fail_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == kAttnWarps) {
    // ================= copy warp =================
    // The split's block-table entries first (one read each, instead of a dependent global load in front of every
    // stage), then stage after stage: wait until the four arithmetic warps have released the slot, issue one bulk
    // copy per page for K and one for V (lane = page; KH heads each), all landing on the slot's barrier.
    const int pg0 = t0 >> log2P, npages = ((t1 - 1) >> log2P) - pg0 + 1;
    const bool cached = npages <= kBtCache;
    if (cached)
      for (int k = lane; k < npages; k += 32) bt_s[k] = __ldg(btb + pg0 + k);
    __syncwarp();
    const uint32_t copy_bytes = (uint32_t)(KH * D * sizeof(half)) << log2P;
    for (int i = 0; i < ntiles; ++i) {
      const int slot = i % NS;
      if (i >= NS && !bar_wait(&empty[slot], (uint32_t)(i / NS - 1) & 1u, kWaitLimit)) {
        fail_s = 1;   // the arithmetic warps find out when their own wait for this stage runs out
        break;
      }
      const int tok0 = i * TS;   // relative to t0
      const int npg = min(TS >> log2P, (t1 - t0 - tok0 + pmask) >> log2P);
      if (lane == 0)
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(sm_u32(&full[slot])),
                     "r"(2u * npg * copy_bytes)
                     : "memory");
      __syncwarp();
      if (lane < 2 * npg) {
        const int isv = lane >= npg, pg = lane - isv * npg, k = (tok0 >> log2P) + pg;
        const int phys = cached ? bt_s[k] : __ldg(btb + pg0 + k);
        const size_t off = (((size_t)phys * n_kv + kvh0) << log2P) * D;
        const half* src = (isv ? vc : kc) + off;
        half* dst = ring + (size_t)slot * 2 * HALF_STAGE + (isv ? HALF_STAGE : 0) + (((size_t)pg * KH) << log2P) * D;
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         sm_u32(dst)),
                     "l"(src), "r"(copy_bytes), "r"(sm_u32(&full[slot]))
                     : "memory");
      }
    }
    return;
  }

  // ================= arithmetic warps =================
  const int kh = warp % KH, tb = warp / KH;   // kv head of the block's group, 16-token block of the stage
  // element offset, inside the K (or V) part of a stage, of token j's row for this warp's head: pages are stored
  // as they are in the cache, [page][head][slot][dim]
  auto row_of = [&](int j) { return (size_t)(((((j >> log2P) * KH) + kh) << log2P) + (j & pmask)) * D; };
  // Q as A fragments: row g = head g of the group (zero beyond HPG), k-step kk holds dims t D/4 + 4 kk + {0,1 | 2,3}
  uint32_t qa[KS][2];
  const int pos = ctx - 1;
  if (ROPE) {
    // rotate-half RoPE on the fly: dim d pairs with d +- D/2; fp32 math, fp16 result (the rounding of rope_append).
    // This lane's D/4 dims, their partners and the matching cos / sin entries arrive as 16-byte loads, all
    // independent, so the prologue costs one memory round trip.
    constexpr int D4 = D / 4;
    const int qkv_stride = (n_q + 2 * n_kv) * D;
    const half* qh = q + (size_t)b * qkv_stride + ((size_t)(kvh0 + kh) * HPG + (g < HPG ? g : 0)) * D;
    const bool lower = t < 2;                       // this lane's dims lie in the first half of the head
    const int dl0 = (t & 1) * D4;                   // their index among the D/2 rotation pairs
    __align__(16) half own[D4], mate[D4];
    __align__(16) float cs[D4], sn[D4];
#pragma unroll
    for (int v = 0; v < D4 / 8; ++v) {
      reinterpret_cast<uint4*>(own)[v] = *reinterpret_cast<const uint4*>(qh + t * D4 + 8 * v);
      reinterpret_cast<uint4*>(mate)[v] = *reinterpret_cast<const uint4*>(qh + t * D4 + (lower ? D / 2 : -(D / 2)) + 8 * v);
    }
#pragma unroll
    for (int v = 0; v < D4 / 4; ++v) {
      reinterpret_cast<float4*>(cs)[v] = *reinterpret_cast<const float4*>(ra.cos_t + (size_t)pos * (D / 2) + dl0 + 4 * v);
      reinterpret_cast<float4*>(sn)[v] = *reinterpret_cast<const float4*>(ra.sin_t + (size_t)pos * (D / 2) + dl0 + 4 * v);
    }
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      half r[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 4 * kk + e;
        const float a = __half2float(lower ? own[i] : mate[i]), bb = __half2float(lower ? mate[i] : own[i]);
        r[e] = __float2half(lower ? a * cs[i] - bb * sn[i] : bb * cs[i] + a * sn[i]);
      }
      qa[kk][0] = g < HPG ? as_u32(__halves2half2(r[0], r[1])) : 0u;
      qa[kk][1] = g < HPG ? as_u32(__halves2half2(r[2], r[3])) : 0u;
    }
  } else {
    const half* qh = q + ((size_t)b * n_q + (kvh0 + kh) * HPG + (g < HPG ? g : 0)) * D + t * (D / 4);
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
      const uint2 v = *reinterpret_cast<const uint2*>(qh + 4 * kk);
      qa[kk][0] = g < HPG ? v.x : 0u;
      qa[kk][1] = g < HPG ? v.y : 0u;
    }
  }
  // ROPE: where the new token sits. Its block is the last live split (if the context is within the prepared cap),
  // its tile i_new, its row j_new, and the warp that owns that row's 16-token block patches it.
  const int rel_new = pos - t0;
  const bool has_new = ROPE && split == nsplit - 1 && rel_new >= 0 && rel_new < t1 - t0;
  const int i_new = has_new ? rel_new / TS : -1, j_new = has_new ? rel_new % TS : 0;
  const float sl2 = scale * 1.44269504088896340736f;   // scores are kept in units of log2(e)
  float m = -CUDART_INF_F, l = 0.f, acc[NB][4];
#pragma unroll
  for (int j = 0; j < NB; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

  int failed_at = -1;
  for (int i = 0; i < ntiles; ++i) {
    const int slot = i % NS;
    const bool ok = bar_wait(&full[slot], (uint32_t)(i / NS) & 1u, kWaitLimit);
    const half* kt = ring + (size_t)slot * 2 * HALF_STAGE;
    const half* vt = kt + HALF_STAGE;
    const int nt = min(TS, t1 - t0 - i * TS);
    const int tok0 = tb * 16;
    if (ROPE && ok && i == i_new && (j_new >> 4) == tb) {
      // the new token: rotated k and raw v into the stage (the copy brought the slot's old bytes) and into the cache
      const int qkv_stride = (n_q + 2 * n_kv) * D;
      const half* kraw = q + (size_t)b * qkv_stride + ((size_t)n_q + kvh0 + kh) * D;
      const half* vraw = kraw + (size_t)n_kv * D;
      half* krow = const_cast<half*>(kt) + row_of(j_new);
      half* vrow = const_cast<half*>(vt) + row_of(j_new);
      const size_t grow = ((((size_t)__ldg(btb + (pos >> log2P)) * n_kv + kvh0 + kh) << log2P) + (pos & pmask)) * D;
      for (int dl = lane; dl < D / 2; dl += 32) {
        const float a = __half2float(kraw[dl]), bb = __half2float(kraw[dl + D / 2]);
        const float c = ra.cos_t[(size_t)pos * (D / 2) + dl], sv = ra.sin_t[(size_t)pos * (D / 2) + dl];
        const half k0 = __float2half(a * c - bb * sv), k1 = __float2half(bb * c + a * sv);
        const half v0 = vraw[dl], v1 = vraw[dl + D / 2];
        krow[dl] = k0; krow[dl + D / 2] = k1; vrow[dl] = v0; vrow[dl + D / 2] = v1;
        ra.kc_w[grow + dl] = k0; ra.kc_w[grow + dl + D / 2] = k1;
        ra.vc_w[grow + dl] = v0; ra.vc_w[grow + dl + D / 2] = v1;
      }
      __syncwarp();
    }
    if (ok && tok0 < nt) {
      // ---- scores of 16 tokens: two n-blocks of 8
      float s[2][4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
        const uint4* kp = reinterpret_cast<const uint4*>(kt + row_of(tok0 + 8 * nb + g) + t * (D / 4));
#pragma unroll
        for (int c = 0; c < CH; ++c) {
          const uint4 kv = kp[c];
          mma16816(s[nb], qa[2 * c][0], 0u, qa[2 * c][1], 0u, kv.x, kv.y);
          mma16816(s[nb], qa[2 * c + 1][0], 0u, qa[2 * c + 1][1], 0u, kv.z, kv.w);
        }
      }
      // this lane: head g, tokens tok0 + 8 nb + 2 t + {0, 1}; rows at or beyond nt hold stale bytes -> masked
      float sc[4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int e = 0; e < 2; ++e)
          sc[2 * nb + e] = tok0 + 8 * nb + 2 * t + e < nt ? s[nb][e] * sl2 : -CUDART_INF_F;
      float mx = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(m, mx);           // finite: token tok0 is valid
      const float alpha = exp2f(m - mn);       // first stage: 2^(-inf) = 0
      m = mn;
      float p[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) p[e] = exp2f(sc[e] - mn);
      l = l * alpha + (p[0] + p[1]) + (p[2] + p[3]);
#pragma unroll
      for (int j = 0; j < NB; ++j) { acc[j][0] *= alpha; acc[j][1] *= alpha; }
      const uint32_t pa0 = as_u32(__floats2half2_rn(p[0], p[1])), pa2 = as_u32(__floats2half2_rn(p[2], p[3]));
      // ---- output: V rows of tokens 2t, 2t+1 (k-slots 2t, 2t+1) and 8+2t, 9+2t (k-slots 2t+8, 2t+9)
      const int ta = tok0 + 2 * t;
      const half* va = vt + row_of(ta) + 8 * g;       // ta is even and pages hold >= 8 tokens: ta + 1 is in the same page
      const half* vb = vt + row_of(ta + 8) + 8 * g;
#pragma unroll
      for (int c = 0; c < VC; ++c) {
        const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);   // a stale row may hold NaN, and 0 * NaN is NaN: feed zeros
        const uint4 v0 = ta < nt ? *reinterpret_cast<const uint4*>(va + 64 * c) : z4;
        const uint4 v1 = ta + 1 < nt ? *reinterpret_cast<const uint4*>(va + D + 64 * c) : z4;
        const uint4 v2 = ta + 8 < nt ? *reinterpret_cast<const uint4*>(vb + 64 * c) : z4;
        const uint4 v3 = ta + 9 < nt ? *reinterpret_cast<const uint4*>(vb + D + 64 * c) : z4;
        const uint32_t a0[4] = {v0.x, v0.y, v0.z, v0.w}, a1[4] = {v1.x, v1.y, v1.z, v1.w};
        const uint32_t a2[4] = {v2.x, v2.y, v2.z, v2.w}, a3[4] = {v3.x, v3.y, v3.z, v3.w};
#pragma unroll
        for (int i2 = 0; i2 < 4; ++i2) {
          mma16816(acc[8 * c + 2 * i2], pa0, 0u, pa2, 0u, __byte_perm(a0[i2], a1[i2], 0x5410),
                   __byte_perm(a2[i2], a3[i2], 0x5410));
          mma16816(acc[8 * c + 2 * i2 + 1], pa0, 0u, pa2, 0u, __byte_perm(a0[i2], a1[i2], 0x7632),
                   __byte_perm(a2[i2], a3[i2], 0x7632));
        }
      }
    }
    if (!ok) { failed_at = i; break; }   // warp-uniform: every lane polled the same barrier
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(sm_u32(&empty[slot])) : "memory");
  }
  // the four arithmetic warps agree on the outcome (a barrier of their 128 threads that ORs a flag)
  {
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.s32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 1, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(any)
        : "r"((int)(failed_at >= 0)), "n"(kAttnThreads)
        : "memory");
    if (any) {
      // leave only after the copies still in flight have landed (bounded again), and say so
      if (failed_at >= 0 && lane == 0) {
        atomicExch(&g_attn_status, 1);
        for (int k = failed_at; k < min(ntiles, failed_at + NS); ++k)
          bar_wait(&full[k % NS], (uint32_t)(k / NS) & 1u, kWaitLimit);
      }
      asm volatile("bar.sync 1, %0;" ::"n"(kAttnThreads) : "memory");
      if (arrive != nullptr && nsplit > 1 && tid == 0) {   // keep the arrival count whole for the calls that follow
        int* cnt = arrive + (size_t)b * gridDim.x + blockIdx.x;
        if (atomicAdd(cnt, 1) == nsplit - 1) *cnt = 0;
      }
      return;
    }
  }

  // ---- merge the warps of each kv head. acc[j][0..1] = O[head g][dim 64 (j / 8) + 8 (2t + e) + j % 8]
  l += __shfl_xor_sync(0xffffffffu, l, 1);
  l += __shfl_xor_sync(0xffffffffu, l, 2);
  if (t == 0) { wm[warp][g] = m; wl[warp][g] = l; }
  float* wo = reinterpret_cast<float*>(ring_raw);   // [kAttnWarps][8][D]; the ring is free now
#pragma unroll
  for (int j = 0; j < NB; ++j)
#pragma unroll
    for (int e = 0; e < 2; ++e)
      wo[((size_t)warp * 8 + g) * D + 64 * (j / 8) + 8 * (2 * t + e) + (j % 8)] = acc[j][e];
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnThreads) : "memory");
  for (int i = tid; i < KH * HPG * D; i += kAttnThreads) {
    const int hk = i / (HPG * D), h = (i / D) % HPG, d = i % D;   // kv head of the group, query head, dim
    float M = -CUDART_INF_F;
#pragma unroll
    for (int r = 0; r < WPH; ++r) M = fmaxf(M, wm[hk + KH * r][h]);
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int r = 0; r < WPH; ++r) {
      const int w = hk + KH * r;
      const float a = exp2f(wm[w][h] - M);   // a warp that had no token: 2^(-inf) = 0
      o = fmaf(a, wo[((size_t)w * 8 + h) * D + d], o);
      L = fmaf(a, wl[w][h], L);
    }
    const size_t hq = (size_t)b * n_q + (kvh0 + hk) * HPG + h;
    if (nsplit == 1) {
      out[hq * D + d] = __float2half(o / L);
    } else {
      o_part[(hq * max_splits + split) * D + d] = o;
      if (d == 0) {   // the combine step works in natural-log units
        m_part[hq * max_splits + split] = M * 0.69314718055994530942f;
        l_part[hq * max_splits + split] = L;
      }
    }
  }
  if (arrive == nullptr || nsplit == 1) return;   // the combine kernel follows / nothing to combine

  // ---- combine as the last block to arrive: every block of (sequence, kv head) takes a ticket after its partials
  // are out; the one that draws the last ticket merges all splits (nobody waits), then zeroes the count for the next
  // call. Blocks of splits beyond the live context never get here and are not counted.
  __threadfence();
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnThreads) : "memory");
  if (tid == 0) {
    int* cnt = arrive + (size_t)b * gridDim.x + blockIdx.x;
    last_s = atomicAdd(cnt, 1) == nsplit - 1;
    if (last_s) *cnt = 0;
  }
  asm volatile("bar.sync 1, %0;" ::"n"(kAttnThreads) : "memory");
  if (!last_s) return;
  __threadfence();
  for (int i = tid; i < KH * HPG * D; i += kAttnThreads) {
    const int hk = i / (HPG * D), h = (i / D) % HPG, d = i % D;
    const size_t hq = (size_t)b * n_q + (kvh0 + hk) * HPG + h;
    const float* mp = m_part + hq * max_splits;
    const float* lp = l_part + hq * max_splits;
    const float* op = o_part + hq * max_splits * D + d;
    float M = -CUDART_INF_F, L = 0.f, acc_o = 0.f;   // same arithmetic, in the same order, as paged_attn_combine_kernel
#pragma unroll 8
    for (int s = 0; s < nsplit; ++s) {
      const float ms = __ldcg(mp + s), ls = __ldcg(lp + s), os = __ldcg(op + (size_t)s * D);
      const float Mn = fmaxf(M, ms);
      const float a = __expf(M - Mn), c = __expf(ms - Mn);
      L = fmaf(L, a, c * ls);
      acc_o = fmaf(acc_o, a, c * os);
      M = Mn;
    }
    out[hq * D + d] = __float2half(acc_o / L);
  }
}

// Grid (n_q, B), D threads: thread d merges dim d of one head over the live splits.
__global__ void paged_attn_combine_kernel(const float* __restrict__ o_part, const float* __restrict__ m_part,
                                          const float* __restrict__ l_part, const int* __restrict__ pos_ptr, int PS,
                                          int max_splits, int D, half* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int ctx = pos_ptr[b] + 1;
  const int nsplit = min((ctx + PS - 1) / PS, max_splits);
  if (nsplit <= 1) return;  // the partial kernel already wrote `out`
  const size_t hq = (size_t)b * gridDim.x + head;
  const float* m = m_part + hq * max_splits;
  const float* l = l_part + hq * max_splits;
  const float* o = o_part + hq * max_splits * D + d;
  // one pass with a running max: every load of the loop is independent of the arithmetic, so the unrolled body has
  // eight splits' worth of loads in flight instead of one round trip per split
  float M = -CUDART_INF_F, L = 0.f, acc = 0.f;
#pragma unroll 8
  for (int s = 0; s < nsplit; ++s) {
    const float ms = __ldg(m + s), ls = __ldg(l + s), os = __ldg(o + (size_t)s * D);
    const float Mn = fmaxf(M, ms);
    const float a = __expf(M - Mn), c = __expf(ms - Mn);   // first split: e^(-inf) = 0
    L = fmaf(L, a, c * ls);
    acc = fmaf(acc, a, c * os);
    M = Mn;
  }
  out[hq * D + d] = __float2half(acc / L);
}

enum : int { ATTN_REGISTER = 1, ATTN_STAGED = 2, ATTN_MMA = 3 };

template <typename Kern>
static cudaError_t allow_ring(Kern kern, size_t bytes, bool* done) {
  if (*done) return cudaSuccess;   // the ring needs more than the default 48 KB of dynamic shared memory
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) *done = true;
  return e;
}

struct AttnArgs {
  const half *q, *kc, *vc;
  const int* bt;
  int bt_stride;
  const int* pos;
  int n_kv, log2P, PS;
  float scale;
  float *o_part, *m_part, *l_part;
  half* out;
  int max_splits, B;
};

template <int D, int HPG, int KH>
static cudaError_t launch_mma(const AttnArgs& a, int dev, cudaStream_t st) {
  static bool configured[64] = {};
  const cudaError_t e = allow_ring(paged_attn_mma_kernel<D, HPG, KH, false>, attn_ring_bytes<D>(), &configured[dev]);
  if (e != cudaSuccess) return e;
  B200_LAUNCH(paged_attn_mma_kernel<D, HPG, KH, false>, dim3(a.n_kv / KH, a.max_splits, a.B), dim3(kMmaThreads),
              attn_ring_bytes<D>(), st, a.q, a.kc, a.vc, a.bt, a.bt_stride, a.pos, a.n_kv, a.log2P, a.PS, a.scale,
              a.o_part, a.m_part, a.l_part, a.out, a.max_splits, RopeArgs{nullptr, nullptr, nullptr, nullptr},
              (int*)nullptr);
  return cudaPeekAtLastError();
}

// the same kernel with RoPE + KV-append folded in: a.q is the raw qkv vector of the step
template <int D, int HPG>
static cudaError_t launch_mma_rope(const AttnArgs& a, const RopeArgs& r, int* arrive, int dev, cudaStream_t st) {
  static bool configured[64] = {};
  const cudaError_t e = allow_ring(paged_attn_mma_kernel<D, HPG, 1, true>, attn_ring_bytes<D>(), &configured[dev]);
  if (e != cudaSuccess) return e;
  B200_LAUNCH(paged_attn_mma_kernel<D, HPG, 1, true>, dim3(a.n_kv, a.max_splits, a.B), dim3(kMmaThreads),
              attn_ring_bytes<D>(), st, a.q, a.kc, a.vc, a.bt, a.bt_stride, a.pos, a.n_kv, a.log2P, a.PS, a.scale,
              a.o_part, a.m_part, a.l_part, a.out, a.max_splits, r, arrive);
  return cudaPeekAtLastError();
}

template <int D, int HPG>
static cudaError_t launch_partial_for(int kind, const AttnArgs& a, cudaStream_t st) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const dim3 grid(a.n_kv, a.max_splits, a.B);
  if (kind == ATTN_MMA) {
    // One kv head per block. The kernel also runs with 2 or 4 adjacent kv heads per block (fewer, larger copies);
    // on 8 sequences x 8192 tokens that measured the same time, and the smaller grid is slower for one sequence.
    return launch_mma<D, HPG, 1>(a, dev, st);
  }
  if (kind == ATTN_STAGED) {
    static bool configured[64] = {};
    const cudaError_t e = allow_ring(paged_attn_staged_kernel<D, HPG>, attn_ring_bytes<D>(), &configured[dev]);
    if (e != cudaSuccess) return e;
    B200_LAUNCH(paged_attn_staged_kernel<D, HPG>, dim3(grid), dim3(kAttnThreads), attn_ring_bytes<D>(), st, a.q, a.kc,
                a.vc, a.bt, a.bt_stride, a.pos, a.n_kv, a.log2P, a.PS, a.scale, a.o_part, a.m_part, a.l_part, a.out,
                a.max_splits);
  } else {
    B200_LAUNCH(paged_attn_partial_kernel<D, HPG>, dim3(grid), dim3(kAttnThreads), 0, st, a.q, a.kc, a.vc, a.bt,
                a.bt_stride, a.pos, a.n_kv, a.log2P, a.PS, a.scale, a.o_part, a.m_part, a.l_part, a.out,
                a.max_splits);
  }
  return cudaPeekAtLastError();
}

template <int D>
static cudaError_t launch_partial(int hpg, int kind, const AttnArgs& a, cudaStream_t st) {
  switch (hpg) {
    case 1: return launch_partial_for<D, 1>(kind, a, st);
    case 2: return launch_partial_for<D, 2>(kind, a, st);
    case 4: return launch_partial_for<D, 4>(kind, a, st);
    case 8: return launch_partial_for<D, 8>(kind, a, st);
    default: return cudaErrorInvalidValue;
  }
}

// 0, or 1 once a block of the staged kernel gave up waiting for its own copies (its outputs are then invalid).
cudaError_t paged_attention_status(int* code) { return cudaMemcpyFromSymbol(code, g_attn_status, sizeof(int)); }

// version: 1 register-load kernel, 2 ring-staged kernel on the fp32 pipes, 3 ring-staged kernel with the contractions
// on the tensor cores, 0 the library's choice (3). 2 and 3 fall back to 1 for shapes the ring does not cover.
cudaError_t paged_attention_dispatch(int version, const void* q, const void* kc, const void* vc, const int* bt,
                                     int bt_stride, const int* pos, int B, int n_q, int n_kv, int D, int log2P, int PS,
                                     int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                     cudaStream_t st) {
  const int hpg = n_q / n_kv;
  const float scale = 1.0f / sqrtf((float)D);
  // the ring-staged kernel copies whole pages: pages of 8..64 tokens, splits that begin on a page boundary
  const bool ring_ok = log2P >= 3 && log2P <= 6 && PS % (1 << log2P) == 0;
  int kind = version == 0 ? ATTN_MMA : version;
  if (!ring_ok) kind = ATTN_REGISTER;
  if (kind == ATTN_MMA && (reinterpret_cast<uintptr_t>(q) & 7u)) kind = ATTN_STAGED;   // Q fragments: 8-byte loads
  const AttnArgs a = {(const half*)q, (const half*)kc, (const half*)vc, bt, bt_stride, pos, n_kv, log2P, PS, scale,
                      o_part, m_part, l_part, (half*)out, max_splits, B};
  cudaError_t e = D == 64 ? launch_partial<64>(hpg, kind, a, st) : launch_partial<128>(hpg, kind, a, st);
  if (e != cudaSuccess) return e;
  if (max_splits > 1) {
    B200_LAUNCH(paged_attn_combine_kernel, dim3(n_q, B), dim3(D), 0, st, o_part, m_part, l_part, pos, PS, max_splits,
                D, (half*)out);
    e = cudaPeekAtLastError();
  }
  return e;
}

cudaError_t rope_append_dispatch(void* qkv, const float* cos_t, const float* sin_t, const int* pos, const int* bt,
                                 int bt_stride, void* kc, void* vc, int B, int n_q, int n_kv, int D, int log2P,
                                 cudaStream_t st);

// RoPE + KV-append + attention (+ combine) for one sequence. Where the ring kernel does not apply (page or split
// size), the two stand-alone kernels run one after the other: same result, one launch more. arrive: nullptr, or
// n_kv zeroed ints - the combine then happens inside the attention kernel (one launch in all).
cudaError_t rope_paged_attention_dispatch(void* qkv, const float* cos_t, const float* sin_t, void* kc, void* vc,
                                          const int* bt, const int* pos, int n_q, int n_kv, int D, int log2P, int PS,
                                          int max_splits, float* o_part, float* m_part, float* l_part, void* out,
                                          int* arrive, cudaStream_t st) {
  const int hpg = n_q / n_kv;
  const bool ring_ok = log2P >= 3 && log2P <= 6 && PS % (1 << log2P) == 0;
  if (!ring_ok) {
    const cudaError_t e = rope_append_dispatch(qkv, cos_t, sin_t, pos, bt, 1 << 30, kc, vc, 1, n_q, n_kv, D, log2P, st);
    if (e != cudaSuccess) return e;
    return paged_attention_dispatch(0, qkv, kc, vc, bt, 1 << 30, pos, 1, n_q, n_kv, D, log2P, PS, max_splits, o_part,
                                    m_part, l_part, out, st);
  }
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  const AttnArgs a = {(const half*)qkv, (const half*)kc, (const half*)vc, bt, 1 << 30, pos, n_kv, log2P, PS,
                      1.0f / sqrtf((float)D), o_part, m_part, l_part, (half*)out, max_splits, 1};
  const RopeArgs r = {cos_t, sin_t, (half*)kc, (half*)vc};
  cudaError_t e = cudaErrorInvalidValue;
#define B200_ROPE_CASE(DD, H) \
  if (D == DD && hpg == H) e = launch_mma_rope<DD, H>(a, r, arrive, dev, st);
  B200_ROPE_CASE(64, 1) B200_ROPE_CASE(64, 2) B200_ROPE_CASE(64, 4) B200_ROPE_CASE(64, 8)
  B200_ROPE_CASE(128, 1) B200_ROPE_CASE(128, 2) B200_ROPE_CASE(128, 4) B200_ROPE_CASE(128, 8)
#undef B200_ROPE_CASE
  if (e != cudaSuccess) return e;
  if (max_splits > 1 && arrive == nullptr) {   // with an arrival array the last block of each head has combined
    B200_LAUNCH(paged_attn_combine_kernel, dim3(n_q, 1), dim3(D), 0, st, o_part, m_part, l_part, pos, PS, max_splits, D,
                (half*)out);
    e = cudaPeekAtLastError();
  }
  return e;
}

}  // namespace b200

// ---- attention without any allocation by the caller --------------------------------------------------------------------
// b200_paged_attention needs three scratch arrays for the split-K partials, and its callers get them from
// cudaMalloc (or torch). Some callers cannot allocate device memory at all: a plugin running inside a host
// application that owns the allocator and hands out nothing, code on a latency-critical path where an allocation may
// synchronise the device, a process whose memory budget was fixed at start-up. For them the partials live in this
// file-scope device array instead. Every GPU that loads the library holds it until the process exits.
//   capacity: 64 query heads x 32 splits x head_dim 128 (about 1 MB), one sequence per call.
// The array is shared by every call on the device and keeps whatever the previous call left; nothing in it has to
// start at zero (the combine step reads only the slots the partial kernel of the same call has just written), so it
// is never cleared. Two calls that overlap on the GPU (different streams) would overwrite each other's partials.
#include "../../include/b200decode.h"

namespace {
constexpr int kNoAllocMaxHeads = 64, kNoAllocMaxSplits = 32, kNoAllocMaxD = 128;
constexpr size_t kNoAllocO = (size_t)kNoAllocMaxHeads * kNoAllocMaxSplits * kNoAllocMaxD;
constexpr size_t kNoAllocML = (size_t)kNoAllocMaxHeads * kNoAllocMaxSplits;
static __device__ __align__(256) float g_attn_scratch[kNoAllocO + 2 * kNoAllocML];

constexpr int kMaxDevices = 64;
float* g_attn_scratch_ptr[kMaxDevices] = {};   // device address of the array, per device, filled on first use
}  // namespace

namespace b200 {
void record_cuda_error(cudaError_t e);   // c_api.cu: what b200_last_cuda_error() reports
}

extern "C" int b200_paged_attention_noalloc(const void* q, const void* kc, const void* vc, const int* bt, const int* pos,
                                            int n_q, int n_kv, int D, int log2P, int PS, int max_splits, void* out,
                                            void* stream) {
  if (!q || !kc || !vc || !bt || !pos || !out || n_q <= 0 || n_kv <= 0 || PS <= 0 || max_splits <= 0 || log2P < 0 ||
      log2P >= 16)
    return B200_ERR_ARG;
  if ((D != 64 && D != 128) || n_q % n_kv) return B200_ERR_SHAPE;
  const int hpg = n_q / n_kv;
  if (hpg != 1 && hpg != 2 && hpg != 4 && hpg != 8) return B200_ERR_SHAPE;
  if (n_q > kNoAllocMaxHeads || max_splits > kNoAllocMaxSplits || D > kNoAllocMaxD) return B200_ERR_LIMIT;
  if ((reinterpret_cast<uintptr_t>(kc) & 15u) || (reinterpret_cast<uintptr_t>(vc) & 15u)) return B200_ERR_ALIGN;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    b200::record_cuda_error(e);
    return B200_ERR_LAUNCH;
  }
  if (dev < 0 || dev >= kMaxDevices) return B200_ERR_LIMIT;
  if (!g_attn_scratch_ptr[dev]) {
    // In host code `g_attn_scratch` is only a handle for the symbol, not a device address: ask the runtime for the
    // address on the current device, once per device.
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_attn_scratch);
    if (e != cudaSuccess || !p) {
      b200::record_cuda_error(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
      return B200_ERR_LAUNCH;
    }
    g_attn_scratch_ptr[dev] = p;
  }
  float* o_part = g_attn_scratch_ptr[dev];
  float* m_part = o_part + (size_t)n_q * max_splits * D;
  float* l_part = m_part + (size_t)n_q * max_splits;
  e = b200::paged_attention_dispatch(0, q, kc, vc, bt, 1 << 30, pos, 1, n_q, n_kv, D, log2P, PS, max_splits, o_part,
                                     m_part, l_part, out, reinterpret_cast<cudaStream_t>(stream));
  if (e == cudaSuccess) return B200_OK;
  b200::record_cuda_error(e);
  return B200_ERR_LAUNCH;
}
