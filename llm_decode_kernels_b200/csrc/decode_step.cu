// One persistent kernel for the whole batch-1 decode step (all layers, LM head, greedy argmax).
//
// Why: at TinyLlama size the step streams 0.55 GB of INT4 weights, 86 us at the B200's measured HBM bandwidth,
// while the same step as 225 separate launches (the reference's structure, runtime/model.py:216-233) costs ~900 us
// of launch and pipeline-drain latency. Here one CTA per SM stays resident for the whole step:
//
//   * a producer warp streams this CTA's slice of every weight matrix, in the order the step consumes them, into a
//     shared-memory ring with 1-D bulk async copies (cp.async.bulk + mbarrier transaction counts). Weights do not
//     depend on activations, so the producer runs ahead of the computation by the depth of the ring and HBM
//     never idles while CTAs wait for each other;
//   * 16 consumer warps do the arithmetic out of the ring: one warp per pair of output rows, x staged once per
//     phase in shared memory (pre-scaled for dot_word), fp32 accumulation, warp-shuffle reduction;
//   * CTAs exchange activation vectors through global memory WITHOUT grid barriers: every fp16 result is stored
//     as a 32-bit word (tag << 16 | value) whose tag is this step's epoch; a consumer polls the words it needs until
//     all carry the current tag. One store + one load crosses the chip instead of fence + atomic + poll + load.
//     Every CTA keeps its own copy of the residual stream in shared memory and redoes the (tiny) residual add and
//     RMSNorm, so those never touch global memory.
//
// Phases per layer (the reference's operator order, with the same rounding points as its fused kernels):
//   A  resid += down[l-1] (layer 0: resid = embedding row);  xin = RMSNorm(resid) * ln1;  qkv = Wqkv xin
//   B  attention: CTA h < n_q takes query head h: RoPE on q and k, append k, v to the paged cache, softmax(q K^T) V
//      over the cache plus the new token
//   C  o = Wo attn
//   D  resid += o;  xin = RMSNorm(resid) * ln2;  act = SwiGLU(Wgate xin, Wup xin)   (gate row i and up row i on one warp)
//   E  down = Wdown act
// then resid += down;  xin = RMSNorm(resid) * norm_f;  logits = Whead xin;  per-CTA argmax candidates; CTA 0 merges
// them (lowest index wins ties), writes tok, history[pos], pos + 1 and the new epoch.
//
// Every wait (mbarrier or tag poll) is bounded. A wait that runs out records a code in StepCtrl::error, raises an
// abort flag that all later waits honour at once, and the CTA leaves after its copies in flight have landed; the
// host reads the code after the step. Nothing here can spin forever.
#include "common.cuh"
#include "decode_step.h"
#include <math_constants.h>

namespace b200 {

namespace {

constexpr int kNCW = 16;                    // consumer warps
constexpr int kNT = kNCW * 32;              // consumer threads
constexpr int kThreads = kNT + 32;          // + producer warp
constexpr int kMaxStages = 16;
constexpr int kSpinLimit = 1 << 18;         // polls / try_waits before a wait gives up (tens of milliseconds)
constexpr int kHeaderBytes = 1024;

enum : int { ERR_POLL = 1, ERR_FULL = 2, ERR_EMPTY = 3, ERR_DRAIN = 4 };

// ---- PTX wrappers --------------------------------------------------------------------------------------------
DEVI uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
DEVI void mbar_init(uint64_t* b, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(count));
}
DEVI void mbar_arrive(uint64_t* b) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(b)) : "memory");
}
DEVI void mbar_expect_tx(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
DEVI bool mbar_try_wait(uint64_t* b, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(b)), "r"(parity)
      : "memory");
  return ok != 0;
}
DEVI void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
DEVI void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kNT) : "memory"); }
// Barrier over the consumer threads that also ORs a flag: every thread gets the same answer, so the decision to
// leave the kernel is taken by all consumer threads together (a thread that left alone would strand the others
// at the next barrier).
DEVI bool consumer_sync_or(int flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.s32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(flag), "n"(kNT)
      : "memory");
  return r != 0;
}
DEVI uint4 ld_poll4(const uint32_t* p) {
  uint4 r;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
DEVI uint2 ld_poll2(const uint32_t* p) {
  uint2 r;
  asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
DEVI void st_tagged(uint32_t* p, uint32_t v) { asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
DEVI void st_tagged2(uint32_t* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// ---- shared state of one CTA -----------------------------------------------------------------------------------
struct Cta {
  uint64_t* full;
  uint64_t* empty;
  volatile int* abort;   // shared-memory flag, CTA-wide
  float* red;            // kNCW + 16 floats of reduction scratch
  half* resid;           // [H] residual stream, private copy
  uint4* xin;            // [Kmax / 8] activations of the running GEMV, pre-scaled for dot_word
  float* att;            // attention scratch
  uint8_t* ring;
  StepCtrl* ctrl;
  uint32_t tagw;         // (tag << 16)
  int ns;                // ring stages
  int stage_bytes, sz_off;
};

DEVI void raise(const Cta& c, int code) {
  if (!*c.abort) {
    *c.abort = 1;
    atomicCAS(&c.ctrl->error, 0, code);
    c.ctrl->abort = 1;
  }
}

// Wait for a ring barrier phase. Returns false (and raises) if the bound is hit or the step is already aborting.
DEVI bool wait_bar(const Cta& c, uint64_t* bar, uint32_t parity, int code) {
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*c.abort) return false;
  }
  raise(c, code);
  return false;
}

// Poll 4 tagged words until all carry this step's tag; returns the 4 fp16 payloads packed as 2 x half2.
DEVI uint2 poll4(const Cta& c, const uint32_t* p) {
  uint4 v = ld_poll4(p);
  int spins = 0;
  while ((((v.x ^ c.tagw) | (v.y ^ c.tagw) | (v.z ^ c.tagw) | (v.w ^ c.tagw)) >> 16) != 0) {
    if (*c.abort) break;
    if (++spins > kSpinLimit) { raise(c, ERR_POLL); break; }
    if ((spins & 255) == 0 && ((volatile StepCtrl*)c.ctrl)->abort) { *c.abort = 1; break; }
    v = ld_poll4(p);
  }
  return make_uint2((v.x & 0xFFFFu) | (v.y << 16), (v.z & 0xFFFFu) | (v.w << 16));
}

DEVI float consumer_sum(const Cta& c, float v, int tid) {
  v = warp_sum(v);
  if ((tid & 31) == 0) c.red[tid >> 5] = v;
  consumer_sync();
  float t = 0.f;
#pragma unroll
  for (int k = 0; k < kNCW; ++k) t += c.red[k];
  consumer_sync();
  return t;
}
DEVI float consumer_max(const Cta& c, float v, int tid) {
  v = warp_max(v);
  if ((tid & 31) == 0) c.red[tid >> 5] = v;
  consumer_sync();
  float t = -CUDART_INF_F;
#pragma unroll
  for (int k = 0; k < kNCW; ++k) t = fmaxf(t, c.red[k]);
  consumer_sync();
  return t;
}

// 4 activations (2 x half2) -> the pre-scaled form dot_word expects: pair 0 times 1/16, pair 1 times 1/256.
DEVI uint2 prescale4(uint2 v) {
  const half2 c_lo = __float2half2_rn(1.0f / 16.0f), c_hi = __float2half2_rn(1.0f / 256.0f);
  return make_uint2(as_u32(__hmul2(as_h2(v.x), c_lo)), as_u32(__hmul2(as_h2(v.y), c_hi)));
}

// ---- x staging ---------------------------------------------------------------------------------------------------
// xin <- prescale(E[0..n)), E tagged. n % 4 == 0.
DEVI void stage_x_plain(const Cta& c, const uint32_t* E, int n, int tid) {
  uint2* xo = reinterpret_cast<uint2*>(c.xin);
  for (int g = tid; g < (n >> 2); g += kNT) xo[g] = prescale4(poll4(c, E + 4 * g));
  consumer_sync();
}

// resid <- resid + delta (delta tagged; or resid <- emb row when E == nullptr), then
// xin <- prescale(w * half(float(resid) * rsqrt(mean(resid^2) + eps))).  H % 4 == 0.
DEVI void stage_x_norm(const Cta& c, const uint32_t* E, const half* emb_row, const half* w, int H, float eps,
                       int tid) {
  uint2* rs = reinterpret_cast<uint2*>(c.resid);
  const uint2* wg = reinterpret_cast<const uint2*>(w);
  float ss = 0.f;
  for (int g = tid; g < (H >> 2); g += kNT) {
    uint2 r;
    if (E) {
      const uint2 d = poll4(c, E + 4 * g);
      r = rs[g];
      r.x = as_u32(__hadd2(as_h2(r.x), as_h2(d.x)));
      r.y = as_u32(__hadd2(as_h2(r.y), as_h2(d.y)));
    } else {
      r = __ldg(reinterpret_cast<const uint2*>(emb_row) + g);
    }
    rs[g] = r;
    const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
    ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ss))));
  }
  const float tot = consumer_sum(c, ss, tid);
  const float rinv = rsqrtf(tot / (float)H + eps);
  uint2* xo = reinterpret_cast<uint2*>(c.xin);
  for (int g = tid; g < (H >> 2); g += kNT) {
    const uint2 r = rs[g];   // this thread's own writes
    const uint2 wv = __ldg(wg + g);
    const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
    uint2 o;
    o.x = as_u32(__hmul2(as_h2(wv.x), __floats2half2_rn(a.x * rinv, a.y * rinv)));
    o.y = as_u32(__hmul2(as_h2(wv.y), __floats2half2_rn(b.x * rinv, b.y * rinv)));
    xo[g] = prescale4(o);
  }
  consumer_sync();
}

// ---- GEMV phase -----------------------------------------------------------------------------------------------------
struct Mat {
  const uint8_t* w;    // packed int4 rows, K/2 bytes each
  const uint8_t* sz;   // (scale, zero) half2 per group, ng * 4 bytes per row
  int N, K;            // N rows (for gate|up: N = I units, rows i and I + i)
  int gu;              // 1: gate|up pairing
};

struct Slice { int ub, ue, ups, nstages, rowbytes, szrow; };

DEVI Slice slice_of(const Mat& m, int log2G, int stage_w, int cta, int ncta) {
  Slice s;
  s.rowbytes = m.K >> 1;
  s.szrow = (m.K >> log2G) << 2;
  const int units = m.gu ? m.N : (m.N + 1) >> 1;
  const int base = units / ncta, rem = units % ncta;
  s.ub = cta * base + min(cta, rem);
  s.ue = s.ub + base + (cta < rem ? 1 : 0);
  s.ups = max(1, stage_w / (2 * s.rowbytes));
  s.nstages = (s.ue - s.ub + s.ups - 1) / s.ups;
  return s;
}

// Producer: issue every stage of one matrix slice. `it` is the running stage counter of the whole step.
DEVI void produce(const Cta& c, const Mat& m, const Slice& s, int& it, int lane) {
  for (int st = 0; st < s.nstages; ++st, ++it) {
    const int slot = it % c.ns;
    const uint32_t parity = ((it / c.ns) & 1) ^ 1;   // a fresh barrier passes the first round
    if (!wait_bar(c, &c.empty[slot], parity, ERR_EMPTY)) return;
    if (lane == 0) {
      const int u0 = s.ub + st * s.ups, u1 = min(s.ue, u0 + s.ups);
      uint8_t* dst = c.ring + (size_t)slot * c.stage_bytes;
      if (m.gu) {
        const int nu = u1 - u0;
        const uint32_t wb = nu * s.rowbytes, sb = nu * s.szrow;
        mbar_expect_tx(&c.full[slot], 2 * (wb + sb));
        bulk_g2s(dst, m.w + (size_t)u0 * s.rowbytes, wb, &c.full[slot]);
        bulk_g2s(dst + wb, m.w + (size_t)(m.N + u0) * s.rowbytes, wb, &c.full[slot]);
        bulk_g2s(dst + c.sz_off, m.sz + (size_t)u0 * s.szrow, sb, &c.full[slot]);
        bulk_g2s(dst + c.sz_off + sb, m.sz + (size_t)(m.N + u0) * s.szrow, sb, &c.full[slot]);
      } else {
        const int r0 = 2 * u0, r1 = min(m.N, 2 * u1);
        const uint32_t wb = (r1 - r0) * s.rowbytes, sb = (r1 - r0) * s.szrow;
        mbar_expect_tx(&c.full[slot], wb + sb);
        bulk_g2s(dst, m.w + (size_t)r0 * s.rowbytes, wb, &c.full[slot]);
        bulk_g2s(dst + c.sz_off, m.sz + (size_t)r0 * s.szrow, sb, &c.full[slot]);
      }
    }
  }
}

// Two rows against xin; returns both fp32 dot products in every lane.
DEVI void dot_two_rows(const Cta& c, const uint4* w0, const uint4* w1, const half2* z0, const half2* z1, int U,
                       int log2G, int lane, float& y0, float& y1) {
  const half2 k1024 = __float2half2_rn(1024.f), k16 = __float2half2_rn(16.f), zero2 = __float2half2_rn(0.f);
  float a0 = 0.f, a1 = 0.f;
#pragma unroll 2
  for (int u = lane; u < U; u += 32) {
    const uint4 wa = w0[u], wb = w1[u];
    const uint4 xa = c.xin[4 * u], xb = c.xin[4 * u + 1], xc = c.xin[4 * u + 2], xd = c.xin[4 * u + 3];
    const int g = (u << 5) >> log2G;
    const half2 sa = z0[g], sb = z1[g];
    {
      const half2 z2 = __half2half2(__high2half(sa));
      const half2 zl = __hadd2(z2, k1024), zh = __hfma2(z2, k16, k1024);
      const half2 p0 = dot_word(wa.x, xa.x, xa.y, xa.z, xa.w, zl, zh, zero2);
      const half2 p1 = dot_word(wa.y, xb.x, xb.y, xb.z, xb.w, zl, zh, zero2);
      const half2 p2 = dot_word(wa.z, xc.x, xc.y, xc.z, xc.w, zl, zh, zero2);
      const half2 p3 = dot_word(wa.w, xd.x, xd.y, xd.z, xd.w, zl, zh, zero2);
      const float2 f = __half22float2(__hadd2(__hadd2(p0, p1), __hadd2(p2, p3)));
      a0 = fmaf(f.x + f.y, __low2float(sa), a0);
    }
    {
      const half2 z2 = __half2half2(__high2half(sb));
      const half2 zl = __hadd2(z2, k1024), zh = __hfma2(z2, k16, k1024);
      const half2 p0 = dot_word(wb.x, xa.x, xa.y, xa.z, xa.w, zl, zh, zero2);
      const half2 p1 = dot_word(wb.y, xb.x, xb.y, xb.z, xb.w, zl, zh, zero2);
      const half2 p2 = dot_word(wb.z, xc.x, xc.y, xc.z, xc.w, zl, zh, zero2);
      const half2 p3 = dot_word(wb.w, xd.x, xd.y, xd.z, xd.w, zl, zh, zero2);
      const float2 f = __half22float2(__hadd2(__hadd2(p0, p1), __hadd2(p2, p3)));
      a1 = fmaf(f.x + f.y, __low2float(sb), a1);
    }
  }
  y0 = warp_sum(a0) * kDotWordRescale;
  y1 = warp_sum(a1) * kDotWordRescale;
}

enum : int { OUT_TAGGED = 0, OUT_SWIGLU = 1, OUT_LOGITS = 2 };

// Consumer side of one matrix slice. OUT_TAGGED: E[row] <- tagged y. OUT_SWIGLU: E[i] <- tagged
// half(silu(gate_i)) * up_i. OUT_LOGITS: logits[row] <- y, and (best, best_idx) track this warp's maximum.
template <int OUT>
DEVI void consume(const Cta& c, const Mat& m, const Slice& s, int log2G, int& it, uint32_t* E, half* logits,
                  unsigned long long& best, int warp, int lane) {
  const int U = m.K >> 5;
  for (int st = 0; st < s.nstages; ++st, ++it) {
    const int slot = it % c.ns;
    const bool ok = wait_bar(c, &c.full[slot], (it / c.ns) & 1, ERR_FULL);
    const int u0 = s.ub + st * s.ups, u1 = min(s.ue, u0 + s.ups), nu = u1 - u0;
    const uint8_t* base = c.ring + (size_t)slot * c.stage_bytes;
    if (ok) {
      for (int j = (warp - (st * s.ups) % kNCW + kNCW) % kNCW; j < nu; j += kNCW) {   // unit -> warp round robin across stages
        int slot0, slot1, row0, row1;
        if (m.gu) { slot0 = j; slot1 = nu + j; row0 = u0 + j; row1 = m.N + u0 + j; }
        else { slot0 = 2 * j; row0 = 2 * (u0 + j); row1 = row0 + 1; slot1 = row1 < m.N ? slot0 + 1 : slot0; }
        float y0, y1;
        dot_two_rows(c, reinterpret_cast<const uint4*>(base + (size_t)slot0 * s.rowbytes),
                     reinterpret_cast<const uint4*>(base + (size_t)slot1 * s.rowbytes),
                     reinterpret_cast<const half2*>(base + c.sz_off + (size_t)slot0 * s.szrow),
                     reinterpret_cast<const half2*>(base + c.sz_off + (size_t)slot1 * s.szrow), U, log2G, lane, y0,
                     y1);
        if (lane == 0) {
          const half h0 = __float2half(y0), h1 = __float2half(y1);
          if (OUT == OUT_SWIGLU) {
            const float gf = __half2float(h0);
            const half sl = __float2half(gf / (1.f + expf(-gf)));
            st_tagged(E + row0, c.tagw | (uint32_t)__half_as_ushort(__hmul(sl, h1)));
          } else if (OUT == OUT_TAGGED) {
            if (row1 < m.N) st_tagged2(E + row0, c.tagw | (uint32_t)__half_as_ushort(h0),
                                       c.tagw | (uint32_t)__half_as_ushort(h1));
            else st_tagged(E + row0, c.tagw | (uint32_t)__half_as_ushort(h0));
          } else {
            logits[row0] = h0;
            if (!__hisnan(h0)) { const unsigned long long k = argmax_key(h0, row0); best = k > best ? k : best; }
            if (row1 < m.N) {
              logits[row1] = h1;
              if (!__hisnan(h1)) { const unsigned long long k = argmax_key(h1, row1); best = k > best ? k : best; }
            }
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
}

// ---- attention for one query head -------------------------------------------------------------------------------------
// All consumer threads of the CTA. q, k, v of this step come from the tagged qkv exchange; tokens 0..pos-1 from the cache.
template <int D>
DEVI void attention_head(const Cta& c, const StepParams& p, const StepLayer& ly, const uint32_t* Eqkv, uint32_t* Eattn,
                         int h, int pos, int tid) {
  constexpr int D2 = D / 2, G4 = D / 4;
  const int hpg = p.n_q / p.n_kv, kvh = h / hpg;
  float* qf = c.att;                       // [D] rotated q * scale
  half* knew = reinterpret_cast<half*>(c.att + D);        // [D] rotated k of this step
  half* vnew = knew + D;                                   // [D]
  half* raw = vnew + D;                                    // [3 D] un-rotated q, k, v
  float* part = c.att + 4 * D;             // [NTG][D] partial outputs
  float* sc = part + (kNT / D2) * D;       // [ctx] scores, then probabilities
  const int pmask = (1 << p.log2P) - 1;

  if (tid < 3 * G4) {
    const int which = tid / G4, g = tid % G4;
    const int head = which == 0 ? h : (which == 1 ? p.n_q + kvh : p.n_q + p.n_kv + kvh);
    reinterpret_cast<uint2*>(raw)[tid] = poll4(c, Eqkv + (size_t)head * D + 4 * g);
  }
  consumer_sync();
  const int page_new = p.bt[pos >> p.log2P], slot_new = pos & pmask;
  if (tid < D) {
    const int i = tid % D2;
    const float cs = p.cos_t[(size_t)pos * D2 + i], sn = p.sin_t[(size_t)pos * D2 + i];
    const half* src = raw + (tid < D2 ? 0 : D);           // threads [0, D2): q pair i; [D2, D): k pair i
    const float a = __half2float(src[i]), b = __half2float(src[i + D2]);
    const half ra = __float2half(a * cs - b * sn), rb = __float2half(b * cs + a * sn);
    if (tid < D2) {
      const float scale = rsqrtf((float)D);
      qf[i] = __half2float(ra) * scale;
      qf[i + D2] = __half2float(rb) * scale;
    } else {
      knew[i] = ra;
      knew[i + D2] = rb;
      if (h % hpg == 0) {
        half* dst = ly.kc + ((((size_t)page_new * p.n_kv + kvh) << p.log2P) + slot_new) * D;
        dst[i] = ra;
        dst[i + D2] = rb;
      }
    }
  } else if (tid < 2 * D) {
    const int i = tid - D;
    const half v = raw[2 * D + i];
    vnew[i] = v;
    if (h % hpg == 0) ly.vc[((((size_t)page_new * p.n_kv + kvh) << p.log2P) + slot_new) * D + i] = v;
  }
  consumer_sync();

  // scores: one token per thread
  float mx = -CUDART_INF_F;
  for (int t = tid; t <= pos; t += kNT) {
    const uint4* kp = t == pos ? reinterpret_cast<const uint4*>(knew)
                               : reinterpret_cast<const uint4*>(
                                     ly.kc + ((((size_t)p.bt[t >> p.log2P] * p.n_kv + kvh) << p.log2P) + (t & pmask)) * D);
    float s = 0.f;
#pragma unroll
    for (int ch = 0; ch < D / 8; ++ch) {
      float kf[8];
      unpack8(kp[ch], kf);
      const float4 qa = *reinterpret_cast<const float4*>(qf + 8 * ch), qb = *reinterpret_cast<const float4*>(qf + 8 * ch + 4);
      s = fmaf(kf[0], qa.x, fmaf(kf[1], qa.y, fmaf(kf[2], qa.z, fmaf(kf[3], qa.w, s))));
      s = fmaf(kf[4], qb.x, fmaf(kf[5], qb.y, fmaf(kf[6], qb.z, fmaf(kf[7], qb.w, s))));
    }
    sc[t] = s;
    mx = fmaxf(mx, s);
  }
  const float M = consumer_max(c, mx, tid);
  float ls = 0.f;
  for (int t = tid; t <= pos; t += kNT) {
    const float e = __expf(sc[t] - M);
    sc[t] = e;
    ls += e;
  }
  const float Lsum = consumer_sum(c, ls, tid);   // its barriers also publish sc[]

  // output: thread (token group tg, dim pair dp)
  constexpr int NTG = kNT / D2;
  const int dp = tid % D2, tg = tid / D2;
  float o0 = 0.f, o1 = 0.f;
  for (int t = tg; t <= pos; t += NTG) {
    const half* vp = t == pos ? vnew : ly.vc + ((((size_t)p.bt[t >> p.log2P] * p.n_kv + kvh) << p.log2P) + (t & pmask)) * D;
    const float2 vf = __half22float2(*reinterpret_cast<const half2*>(vp + 2 * dp));
    const float pr = sc[t];
    o0 = fmaf(pr, vf.x, o0);
    o1 = fmaf(pr, vf.y, o1);
  }
  part[tg * D + 2 * dp] = o0;
  part[tg * D + 2 * dp + 1] = o1;
  consumer_sync();
  if (tid < D) {
    float o = 0.f;
#pragma unroll
    for (int k = 0; k < NTG; ++k) o += part[k * D + tid];
    st_tagged(Eattn + (size_t)h * D + tid, c.tagw | (uint32_t)__half_as_ushort(__float2half(o / Lsum)));
  }
  consumer_sync();
}

}  // namespace

// ---- the kernel ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const __grid_constant__ StepParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  Cta c;
  c.full = reinterpret_cast<uint64_t*>(smem);
  c.empty = c.full + kMaxStages;
  c.abort = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  c.red = reinterpret_cast<float*>(smem + 2 * kMaxStages * 8 + 16);
  c.resid = reinterpret_cast<half*>(smem + kHeaderBytes);
  c.xin = reinterpret_cast<uint4*>(smem + kHeaderBytes + p.resid_bytes);
  c.att = reinterpret_cast<float*>(smem + kHeaderBytes + p.resid_bytes + p.xin_bytes);
  c.ring = smem + kHeaderBytes + p.resid_bytes + p.xin_bytes + p.att_bytes;
  c.ctrl = p.ctrl;
  c.ns = p.ns;
  c.stage_bytes = p.stage_bytes;
  c.sz_off = p.stage_w;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < p.ns; ++i) { mbar_init(&c.full[i], 1); mbar_init(&c.empty[i], kNCW); }
    *c.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const uint32_t epoch = ((volatile StepCtrl*)p.ctrl)->epoch + 1u;
  c.tagw = ((epoch % 65535u) + 1u) << 16;

  const int n_qkv = (p.n_q + 2 * p.n_kv) * p.D, n_att = p.n_q * p.D;
  const int per_layer = n_qkv + n_att + p.H + p.I + p.H;   // exchange words per layer

  if (warp == kNCW) {
    // ================= producer =================
    int it = 0;
    for (int l = 0; l < p.L && !*c.abort; ++l) {
      const StepLayer& ly = p.layers[l];
      const Mat mats[4] = {{(const uint8_t*)ly.w[0], (const uint8_t*)ly.sz[0], n_qkv, p.H, 0},
                           {(const uint8_t*)ly.w[1], (const uint8_t*)ly.sz[1], p.H, n_att, 0},
                           {(const uint8_t*)ly.w[2], (const uint8_t*)ly.sz[2], p.I, p.H, 1},
                           {(const uint8_t*)ly.w[3], (const uint8_t*)ly.sz[3], p.H, p.I, 0}};
#pragma unroll
      for (int k = 0; k < 4; ++k) produce(c, mats[k], slice_of(mats[k], p.log2G, p.stage_w, cta, ncta), it, lane);
    }
    if (!*c.abort) {
      const Mat head = {(const uint8_t*)p.w_head, (const uint8_t*)p.sz_head, p.V, p.H, 0};
      produce(c, head, slice_of(head, p.log2G, p.stage_w, cta, ncta), it, lane);
    }
    // Leave only when every copy issued has landed: a stage is either consumed (its empty barrier completes) or,
    // if the consumers stopped, still full; waiting on the full barriers of the last `ns` stages covers both.
    if (*c.abort) {
      for (int k = max(0, it - c.ns); k < it; ++k) {
        const int slot = k % c.ns;
        for (int i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(&c.full[slot], (k / c.ns) & 1)) break;
      }
    }
    return;
  }

  // ================= consumers =================
  int it = 0;
  unsigned long long best = 0ull;
  const int pos = p.pos[0];
  const half* emb_row = p.emb + (size_t)p.tok[0] * p.H;
  for (int l = 0; l < p.L; ++l) {
    const StepLayer& ly = p.layers[l];
    uint32_t* E = p.xchg + (size_t)l * per_layer;
    uint32_t *Eqkv = E, *Eatt = E + n_qkv, *Eo = Eatt + n_att, *Eact = Eo + p.H, *Edown = Eact + p.I;
    const Mat m_qkv = {(const uint8_t*)ly.w[0], (const uint8_t*)ly.sz[0], n_qkv, p.H, 0};
    const Mat m_o = {(const uint8_t*)ly.w[1], (const uint8_t*)ly.sz[1], p.H, n_att, 0};
    const Mat m_gu = {(const uint8_t*)ly.w[2], (const uint8_t*)ly.sz[2], p.I, p.H, 1};
    const Mat m_dn = {(const uint8_t*)ly.w[3], (const uint8_t*)ly.sz[3], p.H, p.I, 0};

    // A
    stage_x_norm(c, l == 0 ? nullptr : p.xchg + (size_t)(l - 1) * per_layer + (per_layer - p.H), emb_row, ly.ln1, p.H,
                 p.eps, tid);
    if (consumer_sync_or(*c.abort)) return;
    consume<OUT_TAGGED>(c, m_qkv, slice_of(m_qkv, p.log2G, p.stage_w, cta, ncta), p.log2G, it, Eqkv, nullptr, best,
                        warp, lane);
    if (consumer_sync_or(*c.abort)) return;
    // B
    for (int h = cta; h < p.n_q; h += ncta) {
      if (p.D == 64) attention_head<64>(c, p, ly, Eqkv, Eatt, h, pos, tid);
      else attention_head<128>(c, p, ly, Eqkv, Eatt, h, pos, tid);
      if (consumer_sync_or(*c.abort)) return;
    }
    // C
    stage_x_plain(c, Eatt, n_att, tid);
    if (consumer_sync_or(*c.abort)) return;
    consume<OUT_TAGGED>(c, m_o, slice_of(m_o, p.log2G, p.stage_w, cta, ncta), p.log2G, it, Eo, nullptr, best, warp,
                        lane);
    if (consumer_sync_or(*c.abort)) return;
    // D
    stage_x_norm(c, Eo, nullptr, ly.ln2, p.H, p.eps, tid);
    if (consumer_sync_or(*c.abort)) return;
    consume<OUT_SWIGLU>(c, m_gu, slice_of(m_gu, p.log2G, p.stage_w, cta, ncta), p.log2G, it, Eact, nullptr, best, warp,
                        lane);
    if (consumer_sync_or(*c.abort)) return;
    // E
    stage_x_plain(c, Eact, p.I, tid);
    if (consumer_sync_or(*c.abort)) return;
    consume<OUT_TAGGED>(c, m_dn, slice_of(m_dn, p.log2G, p.stage_w, cta, ncta), p.log2G, it, Edown, nullptr, best,
                        warp, lane);
    if (consumer_sync_or(*c.abort)) return;
  }
  // final norm, LM head, argmax
  stage_x_norm(c, p.xchg + (size_t)(p.L - 1) * per_layer + (per_layer - p.H), nullptr, p.norm_f, p.H, p.eps, tid);
  if (consumer_sync_or(*c.abort)) return;
  const Mat head = {(const uint8_t*)p.w_head, (const uint8_t*)p.sz_head, p.V, p.H, 0};
  consume<OUT_LOGITS>(c, head, slice_of(head, p.log2G, p.stage_w, cta, ncta), p.log2G, it, nullptr, p.logits, best,
                      warp, lane);
  // this CTA's candidate: max over its warps' lane-0 keys
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(c.att);
  if (lane == 0) keys[warp] = best;
  if (consumer_sync_or(*c.abort)) return;
  uint32_t* Earg = p.xchg + (size_t)p.L * per_layer;   // [ncta][4] words: (tag|idx lo16, tag|idx hi16, tag|value, tag)
  if (tid == 0) {
    unsigned long long b = 0ull;
    for (int k = 0; k < kNCW; ++k) b = keys[k] > b ? keys[k] : b;
    const uint32_t idx = 0x7FFFFFFFu - (uint32_t)(b & 0xFFFFFFFFu), val = (uint32_t)(b >> 32) & 0xFFFFu;
    uint32_t* e = Earg + 4 * cta;
    asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(e), "r"(c.tagw | (idx & 0xFFFFu)),
                 "r"(c.tagw | (idx >> 16)), "r"(c.tagw | val), "r"(c.tagw | (b ? 1u : 0u))
                 : "memory");
  }
  if (cta == 0) {
    unsigned long long b = 0ull;
    for (int k = tid; k < ncta; k += kNT) {
      const uint2 v = poll4(c, Earg + 4 * k);   // halves: idx lo, idx hi, value key, valid
      const uint32_t idx = v.x, val = v.y & 0xFFFFu, valid = v.y >> 16;
      if (valid) {
        const unsigned long long key = ((unsigned long long)val << 32) | (uint32_t)(0x7FFFFFFFu - idx);
        b = key > b ? key : b;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, b, o);
      b = other > b ? other : b;
    }
    if (lane == 0) keys[kNCW + warp] = b;
    consumer_sync();
    if (tid == 0 && !*c.abort) {
      for (int k = 0; k < kNCW; ++k) b = keys[kNCW + k] > b ? keys[kNCW + k] : b;
      const long long t = (long long)(0x7FFFFFFF - (int)(b & 0xFFFFFFFFu));
      p.tok[0] = t;
      if (p.history) p.history[pos] = t;
      p.pos[0] = pos + 1;
      p.ctrl->epoch = epoch;
    }
  }
}

size_t decode_step_smem_fixed(const StepParams& p) {
  return (size_t)kHeaderBytes + p.resid_bytes + p.xin_bytes + p.att_bytes;
}
int decode_step_threads() { return kThreads; }
int decode_step_max_stages() { return kMaxStages; }
int decode_step_consumer_threads() { return kNT; }

cudaError_t decode_step_launch(const StepParams& p, int grid, size_t smem, cudaStream_t st) {
  static int configured_for = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_for != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    configured_for = dev;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;   // all CTAs co-resident, or the launch is refused
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, decode_step_kernel, p);
}

}  // namespace b200
