// One persistent kernel for the whole batch-1 decode step (all layers, LM head, greedy argmax).
//
// Why: at TinyLlama size the step streams 0.55 GB of INT4 weights, 86 us at the B200's measured HBM bandwidth,
// while the same step as 225 separate launches (the reference's structure, runtime/model.py:216-233) costs ~900 us
// of launch and pipeline-drain latency. Here one CTA per SM stays resident for the whole step:
//
//   * a producer warp streams this CTA's slice of every weight matrix - and, on the CTAs that do attention, the K/V
//     pages of their head - in the order the step consumes them, into a shared-memory ring with 1-D bulk async
//     copies (cp.async.bulk + mbarrier transaction counts). Neither weights nor cached K/V depend on this step's
//     activations, so the producer runs ahead of the computation by the depth of the ring and HBM never idles
//     while CTAs wait for each other;
//   * 16 consumer warps do the arithmetic out of the ring: one warp per pair of output rows, x staged once per
//     phase in shared memory, fp32 accumulation, warp-shuffle reduction;
//   * CTAs exchange activation vectors through global memory WITHOUT grid barriers: every fp16 result is stored
//     as a 32-bit word (tag << 16 | value) whose tag is this step's epoch; a consumer polls the words it needs until
//     all carry the current tag. One store + one load crosses the chip instead of fence + atomic + poll + load.
//     Every CTA keeps its own copy of the residual stream in shared memory and redoes the (tiny) residual add and
//     RMSNorm, so those never touch global memory.
//
// Inner product without per-weight dequantization. A nibble masked in place is an fp16 SUBNORMAL: bits 0..3 of a
// half are q * 2^-24, bits 4..7 are q * 2^-20. So (word & 0x000F000F) and (word & 0x00F000F0) are ready-made half2
// operands; one shift by 8 exposes the other four nibbles. x is staged multiplied by 2^s (pairs under the low mask)
// or 2^(s-4) (pairs under the high mask), s chosen per phase from max|x| so nothing overflows, which makes every
// product q * x * 2^(s-24). With xsum = sum of x over a 32-weight chunk,
//     sum (q - z) * scale * x = scale * (2^(24-s) * sum q x'  -  z * xsum),
// so the zero point costs one FMA per chunk instead of one subtraction per weight: 9 integer/half2 operations per
// 8 weights in the loop. The per-element weight this stands for is the format's dequantized weight
// (dequant_w4a16 in gemv_w4a16.cu proves the format bit-exactly).
//
// Phases per layer (the reference's operator order, with the same rounding points as its fused kernels):
//   A  resid += down[l-1] (layer 0: resid = embedding row);  x = RMSNorm(resid) * ln1;  qkv = Wqkv x
//   B  attention: CTA h < n_q takes query head h: RoPE on q and k, append k, v to the paged cache, then per-warp
//      online softmax over the cached tokens (from the ring) plus the new token, merged once across warps
//   C  o = Wo attn
//   D  resid += o;  x = RMSNorm(resid) * ln2;  act = SwiGLU(Wgate x, Wup x)   (gate row i and up row i on one warp)
//   E  down = Wdown act
// then resid += down;  x = RMSNorm(resid) * norm_f;  logits = Whead x;  per-CTA argmax candidates; CTA 0 merges
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
constexpr int kHeaderBytes = 2048;
constexpr int kMaxKvTokens = 64;            // cached tokens per ring stage in attention (16 warps x 4 tokens)

enum : int { ERR_POLL = 1, ERR_FULL = 2, ERR_EMPTY = 3 };

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
DEVI void st_tagged(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
DEVI void st_tagged2(uint32_t* p, uint32_t a, uint32_t b) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// ---- shared state of one CTA -----------------------------------------------------------------------------------
struct Cta {
  uint64_t* full;
  uint64_t* empty;
  volatile int* abort;   // shared-memory flag, CTA-wide
  float* red;            // 2 * kNCW floats of reduction scratch
  half* resid;           // [H] residual stream, private copy
  uint4* xin;            // [Kmax / 8] activations of the running GEMV, scaled, 16-byte chunks swizzled (see swz)
  float* xsum;           // [Kmax / 32] sum of the unscaled activations of each 32-weight chunk
  float* att;            // attention scratch
  float* part;           // [rows of the largest slice][segments] partial dot products of the running GEMV
  uint8_t* ring;
  StepCtrl* ctrl;
  uint32_t tagw;         // (tag << 16)
  int ns;                // ring stages
  int nopoll;            // debug: take exchange words as they are (timing experiments only)
  int stage_bytes;
};

DEVI void raise(const Cta& c, int code) {
  if (!*c.abort) {
    *c.abort = 1;
    atomicCAS(&c.ctrl->error, 0, code);
    c.ctrl->abort = 1;
  }
}

// Wait for a ring barrier phase. Returns false (and raises) if the bound is hit or the step is already aborting.
// `nap` nanoseconds of sleep follow every failed attempt: a waiting warp must not eat the issue slots of the warps
// it shares a scheduler with (the producer waits for most of the step).
DEVI bool wait_bar(const Cta& c, uint64_t* bar, uint32_t parity, int code, unsigned nap = 0) {
#pragma unroll 1
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*c.abort) return false;
    if (nap) __nanosleep(nap);
  }
  raise(c, code);
  return false;
}

// Poll 4 tagged words until all carry this step's tag; returns the 4 fp16 payloads packed as 2 x half2.
DEVI uint2 poll4(const Cta& c, const uint32_t* p) {
  uint4 v = ld_poll4(p);
  int spins = 0;
  while (!c.nopoll && ((((v.x ^ c.tagw) | (v.y ^ c.tagw) | (v.z ^ c.tagw) | (v.w ^ c.tagw)) >> 16) != 0)) {
    if (*c.abort) break;
    if (++spins > kSpinLimit) { raise(c, ERR_POLL); break; }
    if ((spins & 255) == 0 && ((volatile StepCtrl*)c.ctrl)->abort) { *c.abort = 1; break; }
    v = ld_poll4(p);
  }
  return make_uint2((v.x & 0xFFFFu) | (v.y << 16), (v.z & 0xFFFFu) | (v.w << 16));
}

// Block-wide (consumer threads) sum and max in one barrier pair.
DEVI void consumer_sum_max(const Cta& c, float s, float m, int tid, float& s_all, float& m_all) {
  s = warp_sum(s);
  m = warp_max(m);
  if ((tid & 31) == 0) { c.red[tid >> 5] = s; c.red[kNCW + (tid >> 5)] = m; }
  consumer_sync();
  float ts = 0.f, tm = 0.f;
#pragma unroll
  for (int k = 0; k < kNCW; ++k) { ts += c.red[k]; tm = fmaxf(tm, c.red[kNCW + k]); }
  consumer_sync();
  s_all = ts;
  m_all = tm;
}

// ---- x staging ---------------------------------------------------------------------------------------------------
// Store granule g (4 activations as 2 x half2, unscaled) scaled into xin and add its sum into xsum (8 granules of
// consecutive threads make one 32-weight chunk).
DEVI void put_granule(const Cta& c, int g, uint2 v, const XScale& sc, int tid) {
  const float2 a = __half22float2(as_h2(v.x)), b = __half22float2(as_h2(v.y));
  float s = (a.x + a.y) + (b.x + b.y);
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if ((tid & 7) == 0) c.xsum[g >> 3] = s;
  uint2 o;
  o.x = as_u32(__hmul2(as_h2(v.x), sc.lo));
  o.y = as_u32(__hmul2(as_h2(v.y), sc.hi));
  reinterpret_cast<uint2*>(c.xin)[2 * swz(g >> 1) + (g & 1)] = o;
}

DEVI float absmax4(uint2 v) {
  const float2 a = __half22float2(__habs2(as_h2(v.x))), b = __half22float2(__habs2(as_h2(v.y)));
  return fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y));
}

// x <- E[0..n) (tagged). n % 32 == 0. Returns the factor that undoes the staging scale.
DEVI float stage_x_plain(const Cta& c, const uint32_t* E, int n, int tid) {
  uint2* raw = reinterpret_cast<uint2*>(c.xin);   // pass 1 parks the unscaled granules at their final place
  float mx = 0.f;
  for (int g = tid; g < (n >> 2); g += kNT) {
    const uint2 v = poll4(c, E + 4 * g);
    raw[2 * swz(g >> 1) + (g & 1)] = v;
    mx = fmaxf(mx, absmax4(v));
  }
  float dummy, xmax;
  consumer_sum_max(c, 0.f, mx, tid, dummy, xmax);
  const XScale sc = scale_for(xmax);
  for (int g = tid; g < (n >> 2); g += kNT) put_granule(c, g, raw[2 * swz(g >> 1) + (g & 1)], sc, tid);
  consumer_sync();
  return sc.resc;
}

// resid <- resid + delta (delta tagged; or resid <- emb row when E == nullptr), then
// x <- w * half(float(resid) * rsqrt(mean(resid^2) + eps)).  H % 32 == 0.
DEVI float stage_x_norm(const Cta& c, const uint32_t* E, const half* emb_row, const half* w, int H, float eps,
                        int tid) {
  uint2* rs = reinterpret_cast<uint2*>(c.resid);
  const uint2* wg = reinterpret_cast<const uint2*>(w);
  float ss = 0.f, mw = 0.f;
  for (int g = tid; g < (H >> 2); g += kNT) {
    const uint2 wv = __ldg(wg + g);   // issued before the poll: its latency hides behind the wait
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
    mw = fmaxf(mw, absmax4(make_uint2(as_u32(__hmul2(as_h2(r.x), as_h2(wv.x))), as_u32(__hmul2(as_h2(r.y), as_h2(wv.y))))));
  }
  float tot, mwall;
  consumer_sum_max(c, ss, mw, tid, tot, mwall);
  const float rinv = rsqrtf(tot / (float)H + eps);
  const XScale sc = scale_for(mwall * rinv * 1.01f);
  for (int g = tid; g < (H >> 2); g += kNT) {
    const uint2 r = rs[g];   // this thread's own writes
    const uint2 wv = __ldg(wg + g);
    const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
    uint2 o;
    o.x = as_u32(__hmul2(as_h2(wv.x), __floats2half2_rn(a.x * rinv, a.y * rinv)));
    o.y = as_u32(__hmul2(as_h2(wv.y), __floats2half2_rn(b.x * rinv, b.y * rinv)));
    put_granule(c, g, o, sc, tid);
  }
  consumer_sync();
  return sc.resc;
}

// One entry point for both kinds of staging (a single call site keeps a single copy of the code).
DEVI float stage_x(const Cta& c, const uint32_t* E, const half* emb_row, const half* nw, int n, float eps, int tid) {
  return nw ? stage_x_norm(c, E, emb_row, nw, n, eps, tid) : stage_x_plain(c, E, n, tid);
}

// ---- GEMV phase -----------------------------------------------------------------------------------------------------
// A weight matrix in "stream layout" (see repack_stream_kernel): for every CTA, for every ring stage of its slice,
// the packed rows of the stage followed by their (scale, zero) rows, contiguous - one bulk copy per stage.
struct Mat {
  const uint8_t* stream;
  int N, K;            // N rows (for gate|up: N = I units, rows i and I + i)
  int gu;              // 1: gate|up pairing
};

struct Slice { int ub, ue, ups, nstages, rowbytes, szrow; };

// Position in the ring. Stages are used strictly in order by producer and consumers alike, so a slot index and a
// parity bit that flips on wrap-around replace a stage counter (and the divisions by the ring size it would need).
struct RingPos {
  int slot;
  uint32_t parity;
  int count;   // stages passed (the producer's abort path needs it)
};
DEVI void advance(RingPos& r, int ns) {
  ++r.count;
  if (++r.slot == ns) { r.slot = 0; r.parity ^= 1u; }
}

// How the consumer warps split a matrix with rows of K weights: see consume().
struct WarpMap { int segs, sper, seg0, group, rank, upsmod; };
DEVI WarpMap warp_map(int K, int ups, int warp) {
  WarpMap w;
  const int U = K >> 5;
  w.segs = (U + 31) >> 5;
  w.sper = (w.segs + kNCW - 1) / kNCW;
  w.seg0 = w.sper == 1 ? warp % w.segs : warp;
  w.group = w.sper == 1 ? (kNCW - w.seg0 + w.segs - 1) / w.segs : 1;
  w.rank = w.sper == 1 ? warp / w.segs : 0;
  w.upsmod = ups % w.group;
  return w;
}

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

// Producer: issue every stage of one matrix slice (one copy each; a bulk copy costs ~0.2 us to issue whatever its
// size, so several small copies per stage would make the producer the bottleneck). `it` is the running stage
// counter of the step.
DEVI void produce(const Cta& c, const Mat& m, const Slice& s, RingPos& rp, int lane) {
  const size_t rowall = (size_t)s.rowbytes + s.szrow;
  for (int st = 0; st < s.nstages; ++st, advance(rp, c.ns)) {
    const int slot = rp.slot;
    if (!wait_bar(c, &c.empty[slot], rp.parity, ERR_EMPTY, 200)) return;
    if (lane == 0) {
      const int u0 = s.ub + st * s.ups, u1 = min(s.ue, u0 + s.ups);
      const int r0 = 2 * u0, r1 = m.gu ? 2 * u1 : min(m.N, 2 * u1);   // gate|up: two rows per unit, always
      const uint32_t bytes = (uint32_t)((r1 - r0) * rowall);
      mbar_expect_tx(&c.full[slot], bytes);
      bulk_g2s(c.ring + (size_t)slot * c.stage_bytes, m.stream + (size_t)r0 * rowall, bytes, &c.full[slot]);
    }
  }
}

// Cached tokens per attention ring stage: K rows in the first half of the stage, V rows in the second.
DEVI int kv_tokens_per_stage(const StepParams& p) {
  int t = min(kMaxKvTokens, p.stage_w / (4 * p.D));
  return t & ~((1 << p.log2P) - 1);
}

// Producer: the cached K/V rows [0, pos) of one kv head, page by page. Whole pages are copied; rows at or beyond
// pos in the last page are ignored by the consumer.
DEVI void produce_kv(const Cta& c, const StepParams& p, const StepLayer& ly, int kvh, int pos, RingPos& rp, int lane) {
  const int tps = kv_tokens_per_stage(p), pps = tps >> p.log2P;
  const uint32_t page_bytes = (uint32_t)(p.D * 2) << p.log2P;
  const int nst = (pos + tps - 1) / tps;
  for (int st = 0; st < nst; ++st, advance(rp, c.ns)) {
    const int slot = rp.slot;
    if (!wait_bar(c, &c.empty[slot], rp.parity, ERR_EMPTY, 200)) return;
    const int pg0 = st * pps, npg = min(pps, ((pos + (1 << p.log2P) - 1) >> p.log2P) - pg0);
    uint8_t* dst = c.ring + (size_t)slot * c.stage_bytes;
    if (lane == 0) mbar_expect_tx(&c.full[slot], 2 * npg * page_bytes);
    __syncwarp();
    if (lane < npg) {
      const size_t off = ((size_t)p.bt[pg0 + lane] * p.n_kv + kvh) * page_bytes;
      bulk_g2s(dst + lane * page_bytes, reinterpret_cast<const uint8_t*>(ly.kc) + off, page_bytes, &c.full[slot]);
      bulk_g2s(dst + (size_t)tps * p.D * 2 + lane * page_bytes, reinterpret_cast<const uint8_t*>(ly.vc) + off,
               page_bytes, &c.full[slot]);
    }
  }
}

DEVI XChunk load_xchunk(const Cta& c, int u) {
  const int sw = (u >> 1) & 3;
  XChunk r;
  r.x0 = c.xin[4 * u + (0 ^ sw)];
  r.x1 = c.xin[4 * u + (1 ^ sw)];
  r.x2 = c.xin[4 * u + (2 ^ sw)];
  r.x3 = c.xin[4 * u + (3 ^ sw)];
  r.xs = c.xsum[u];
  return r;
}

// Sum p0 over the warp and p1 over the warp with 6 shuffles instead of 10: the first exchange leaves the lower
// half-warp holding p0 partials and the upper one p1 partials. Result: lane 0 has sum p0, lane 16 has sum p1.
DEVI float reduce_pair(float p0, float p1, int lane) {
  const bool up = lane & 16;
  float v = up ? p1 : p0;
  v += __shfl_xor_sync(0xffffffffu, up ? p0 : p1, 16);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

enum : int { OUT_TAGGED = 0, OUT_SWIGLU = 1, OUT_LOGITS = 2 };

// Consumer side of one matrix slice. A row is cut into segments of 32 chunks (1024 weights); every warp is bound to
// ONE segment for the whole slice (warp w -> segment w mod segs) and lane l to chunk l of it, so the lane's 32
// activations sit in registers and are loaded once per slice; the warps that share a segment split the units
// (pairs of rows) round robin. Per unit a lane reads two 16-byte weight chunks and two (scale, zero) words, runs the
// 72-instruction core, and the warp leaves two partial sums in shared memory (c.part). After one barrier per slice
// thread i finishes unit i: it adds the segments in a fixed order (deterministic) and emits the output.
// When a row has more than 16 segments (K > 16384) a warp owns several segments and reloads x between them.
//   OUT_TAGGED: E[row] <- tagged y.  OUT_SWIGLU: E[i] <- tagged half(silu(gate_i)) * up_i.
//   OUT_LOGITS: logits[row] <- y, and `best` tracks this thread's maximum.
DEVI void consume(const Cta& c, const Mat& m, const Slice& s, const WarpMap& wm_, int log2G, float resc, RingPos& rp,
                  const int OUT, uint32_t* E, half* logits, unsigned long long& best, int tid) {
  const int lane = tid & 31;
  const int U = m.K >> 5, segs = wm_.segs;
  const int sper = wm_.sper;     // segments per warp (1 unless K > 16384)
  const int seg0 = wm_.seg0;     // first (usually only) segment of this warp
  const int group = wm_.group;   // warps sharing seg0
  const int rank = wm_.rank;     // this warp's place among them
  XChunk x;
  int u = 32 * seg0 + lane;
  if (u < U) x = load_xchunk(c, u);
  const int g = (u << 5) >> log2G;
  int joff = 0;   // (index of the stage's first unit within the slice) mod group
  for (int st = 0; st < s.nstages; ++st, advance(rp, c.ns)) {
    const int slot = rp.slot;
    const bool ok = wait_bar(c, &c.full[slot], rp.parity, ERR_FULL);
    const int u0 = s.ub + st * s.ups, u1 = min(s.ue, u0 + s.ups), nu = u1 - u0;
    const uint8_t* base = c.ring + (size_t)slot * c.stage_bytes;
    const uint8_t* szbase = base + (size_t)((m.gu ? 2 * u1 : min(m.N, 2 * u1)) - 2 * u0) * s.rowbytes;
    if (ok) {
      const int ui0 = u0 - s.ub;   // index of the stage's first unit within the slice
      if (sper == 1) {
        // two units per trip: twice the independent work between dependent shuffles, one combined reduction
        for (int j = rank - joff + (rank < joff ? group : 0); j < nu; j += 2 * group) {
          const int j2 = j + group < nu ? j + group : j;   // second unit of the trip (repeats the first at the tail)
          int sa0, sa1, sb0, sb1;
          if (m.gu) { sa0 = j; sa1 = nu + j; sb0 = j2; sb1 = nu + j2; }
          else {
            sa0 = 2 * j; sa1 = 2 * (u0 + j) + 1 < m.N ? sa0 + 1 : sa0;
            sb0 = 2 * j2; sb1 = 2 * (u0 + j2) + 1 < m.N ? sb0 + 1 : sb0;
          }
          float p0 = 0.f, p1 = 0.f, q0 = 0.f, q1 = 0.f;
          if (u < U) {
            const uint4 wa0 = reinterpret_cast<const uint4*>(base + (size_t)sa0 * s.rowbytes)[u];
            const uint4 wa1 = reinterpret_cast<const uint4*>(base + (size_t)sa1 * s.rowbytes)[u];
            const uint4 wb0 = reinterpret_cast<const uint4*>(base + (size_t)sb0 * s.rowbytes)[u];
            const uint4 wb1 = reinterpret_cast<const uint4*>(base + (size_t)sb1 * s.rowbytes)[u];
            const half2 za0 = reinterpret_cast<const half2*>(szbase + (size_t)sa0 * s.szrow)[g];
            const half2 za1 = reinterpret_cast<const half2*>(szbase + (size_t)sa1 * s.szrow)[g];
            const half2 zb0 = reinterpret_cast<const half2*>(szbase + (size_t)sb0 * s.szrow)[g];
            const half2 zb1 = reinterpret_cast<const half2*>(szbase + (size_t)sb1 * s.szrow)[g];
            chunk_two_rows(wa0, wa1, za0, za1, x, resc, p0, p1);
            if (j2 != j) chunk_two_rows(wb0, wb1, zb0, zb1, x, resc, q0, q1);   // warp-uniform: no second unit at the tail
          }
          // 4 sums with 7 shuffles: quarter q of the warp ends up holding value q
          const int qd = lane >> 3;
          float v0 = (qd & 2) ? q0 : p0, v1 = (qd & 2) ? q1 : p1;          // this half-warp's pair
          const float o0 = (qd & 2) ? p0 : q0, o1 = (qd & 2) ? p1 : q1;    // the other half-warp's pair
          v0 += __shfl_xor_sync(0xffffffffu, o0, 16);
          v1 += __shfl_xor_sync(0xffffffffu, o1, 16);
          float v = (qd & 1) ? v1 : v0;
          v += __shfl_xor_sync(0xffffffffu, (qd & 1) ? v0 : v1, 8);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          if ((lane & 7) == 0) {
            const int jj = (qd & 2) ? j2 : j;
            if (!(qd & 2) || j2 != j) c.part[((ui0 + jj) * 2 + (qd & 1)) * segs + seg0] = v;
          }
        }
      } else {
        for (int j = 0; j < nu; ++j) {
          int slot0, slot1;
          if (m.gu) { slot0 = j; slot1 = nu + j; }
          else { slot0 = 2 * j; slot1 = 2 * (u0 + j) + 1 < m.N ? slot0 + 1 : slot0; }
          const uint4* w0 = reinterpret_cast<const uint4*>(base + (size_t)slot0 * s.rowbytes);
          const uint4* w1 = reinterpret_cast<const uint4*>(base + (size_t)slot1 * s.rowbytes);
          const half2* z0 = reinterpret_cast<const half2*>(szbase + (size_t)slot0 * s.szrow);
          const half2* z1 = reinterpret_cast<const half2*>(szbase + (size_t)slot1 * s.szrow);
          for (int seg = seg0; seg < segs; seg += kNCW) {
            const int uu = 32 * seg + lane;
            float p0 = 0.f, p1 = 0.f;
            if (uu < U) {
              const XChunk xx = load_xchunk(c, uu);
              const int gg = (uu << 5) >> log2G;
              chunk_two_rows(w0[uu], w1[uu], z0[gg], z1[gg], xx, resc, p0, p1);
            }
            const float v = reduce_pair(p0, p1, lane);
            if ((lane & 15) == 0) c.part[((ui0 + j) * 2 + (lane >> 4)) * segs + seg] = v;
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
    joff += wm_.upsmod;
    if (joff >= group) joff -= group;
  }
  consumer_sync();
  for (int i = tid; i < s.ue - s.ub; i += kNT) {
    float y0 = 0.f, y1 = 0.f;
    for (int k = 0; k < segs; ++k) { y0 += c.part[(2 * i) * segs + k]; y1 += c.part[(2 * i + 1) * segs + k]; }
    const half h0 = __float2half(y0), h1 = __float2half(y1);
    const int unit = s.ub + i;
    if (OUT == OUT_SWIGLU) {
      const float gf = __half2float(h0);
      const half sl = __float2half(__fdividef(gf, 1.f + __expf(-gf)));
      st_tagged(E + unit, c.tagw | (uint32_t)__half_as_ushort(__hmul(sl, h1)));
    } else {
      const int row0 = 2 * unit, row1 = row0 + 1;
      if (OUT == OUT_TAGGED) {
        if (row1 < m.N) st_tagged2(E + row0, c.tagw | (uint32_t)__half_as_ushort(h0),
                                   c.tagw | (uint32_t)__half_as_ushort(h1));
        else st_tagged(E + row0, c.tagw | (uint32_t)__half_as_ushort(h0));
      } else {
        logits[row0] = h0;
        if (!__hisnan(h0)) { const unsigned long long key = argmax_key(h0, row0); best = key > best ? key : best; }
        if (row1 < m.N) {
          logits[row1] = h1;
          if (!__hisnan(h1)) { const unsigned long long key = argmax_key(h1, row1); best = key > best ? key : best; }
        }
      }
    }
  }
}

// ---- attention for one query head -------------------------------------------------------------------------------------
// All consumer threads of the CTA. q, k, v of this step come from the tagged qkv exchange, tokens 0..pos-1 from ring
// stages filled by produce_kv. Lane (t = lane >> 3, c = lane & 7) of warp w owns token slot 4 w + t of a stage and
// dims [c D/8, (c+1) D/8) of it; each warp keeps a private online-softmax state, merged once at the end.
template <int D>
DEVI void attention_head(const Cta& c, const StepParams& p, const StepLayer& ly, const uint32_t* Eqkv, uint32_t* Eattn,
                         int h, int pos, float cs, float sn, int page_new, RingPos& rp, int tid) {
  constexpr int D2 = D / 2, G4 = D / 4, DPL = D / 8;
  const int warp = tid >> 5, lane = tid & 31, ts = lane >> 3, ch = lane & 7;
  const int hpg = p.n_q / p.n_kv, kvh = h / hpg;
  float* qf = c.att;                                         // [D] rotated q * 1/sqrt(D)
  half* knew = reinterpret_cast<half*>(c.att + D);           // [D] rotated k of this step
  half* vnew = knew + D;                                     // [D]
  half* raw = vnew + D;                                      // [3 D] un-rotated q, k, v
  float* wo = c.att + 4 * D;                                 // [kNCW][D] per-warp outputs
  float* wm = wo + kNCW * D;                                 // [kNCW] per-warp max
  float* wl = wm + kNCW;                                     // [kNCW] per-warp sum
  const int pmask = (1 << p.log2P) - 1;

  if (tid < 3 * G4) {
    const int which = tid / G4, g = tid % G4;
    const int head = which == 0 ? h : (which == 1 ? p.n_q + kvh : p.n_q + p.n_kv + kvh);
    reinterpret_cast<uint2*>(raw)[tid] = poll4(c, Eqkv + (size_t)head * D + 4 * g);
  }
  consumer_sync();
  if (tid < 2 * D) {
    const int slot_new = pos & pmask;
    const size_t row_new = ((((size_t)page_new * p.n_kv + kvh) << p.log2P) + slot_new) * D;
    if (tid < D) {
      const int i = tid % D2;
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
        if (h % hpg == 0) { ly.kc[row_new + i] = ra; ly.kc[row_new + i + D2] = rb; }
      }
    } else {
      const int i = tid - D;
      const half v = raw[2 * D + i];
      vnew[i] = v;
      if (h % hpg == 0) ly.vc[row_new + i] = v;
    }
  }
  consumer_sync();

  float qreg[DPL];
#pragma unroll
  for (int d = 0; d < DPL; ++d) qreg[d] = qf[ch * DPL + d];
  float m = -CUDART_INF_F, l = 0.f, acc[DPL];
#pragma unroll
  for (int d = 0; d < DPL; ++d) acc[d] = 0.f;

  // fold one token (K row kp, V row vp, both this lane's DPL dims) into the warp's state; `valid` per token slot
  auto fold = [&](const half* kp, const half* vp, bool valid) {
    float kf[DPL], s = 0.f;
#pragma unroll
    for (int d8 = 0; d8 < DPL; d8 += 8) unpack8(*reinterpret_cast<const uint4*>(kp + d8), kf + d8);
#pragma unroll
    for (int d = 0; d < DPL; ++d) s = fmaf(kf[d], qreg[d], s);
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    s = valid ? s : -CUDART_INF_F;
    float mw = fmaxf(s, __shfl_xor_sync(0xffffffffu, s, 8));
    mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
    const float mn = fmaxf(m, mw);
    if (mn == -CUDART_INF_F) return;           // nothing valid yet in this warp (warp-uniform)
    const float alpha = __expf(m - mn), pr = __expf(s - mn);
    m = mn;
    l = l * alpha + pr;
    float vf[DPL];
#pragma unroll
    for (int d8 = 0; d8 < DPL; d8 += 8) unpack8(*reinterpret_cast<const uint4*>(vp + d8), vf + d8);
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[d] = fmaf(pr, vf[d], acc[d] * alpha);
  };

  const int tps = kv_tokens_per_stage(p);
  const int nst = (pos + tps - 1) / tps;
  for (int st = 0; st < nst; ++st, advance(rp, c.ns)) {
    const int slot = rp.slot;
    const bool ok = wait_bar(c, &c.full[slot], rp.parity, ERR_FULL);
    const half* kbase = reinterpret_cast<const half*>(c.ring + (size_t)slot * c.stage_bytes);
    const half* vbase = kbase + (size_t)tps * D;
    const int nt = min(tps, pos - st * tps);
    if (ok) {
      for (int j0 = 4 * warp; j0 < nt; j0 += 4 * kNCW) {
        const int j = j0 + ts;
        const int jj = min(j, nt - 1);
        fold(kbase + (size_t)jj * D + ch * DPL, vbase + (size_t)jj * D + ch * DPL, j < nt);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&c.empty[slot]);
  }
  if (warp == 0) fold(knew + ch * DPL, vnew + ch * DPL, ts == 0);   // the token of this step

  // merge: token slots inside the warp, then the warps
  float lw = l;
  lw += __shfl_xor_sync(0xffffffffu, lw, 8);
  lw += __shfl_xor_sync(0xffffffffu, lw, 16);
#pragma unroll
  for (int d = 0; d < DPL; ++d) {
    acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 8);
    acc[d] += __shfl_xor_sync(0xffffffffu, acc[d], 16);
  }
  if (ts == 0) {
#pragma unroll
    for (int d = 0; d < DPL; ++d) wo[warp * D + ch * DPL + d] = acc[d];
    if (ch == 0) { wm[warp] = m; wl[warp] = lw; }
  }
  consumer_sync();
  if (tid < D) {
    float M = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < kNCW; ++w) M = fmaxf(M, wm[w]);
    float o = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < kNCW; ++w) {
      const float a = __expf(wm[w] - M);   // a warp that saw no token: e^(-inf) = 0
      o = fmaf(a, wo[w * D + tid], o);
      L = fmaf(a, wl[w], L);
    }
    st_tagged(Eattn + (size_t)h * D + tid, c.tagw | (uint32_t)__half_as_ushort(__float2half(o / L)));
  }
  consumer_sync();
}

}  // namespace

// ---- the kernel ------------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const __grid_constant__ StepParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  Cta c;
  c.full = reinterpret_cast<uint64_t*>(smem);
  c.empty = c.full + kMaxStages;
  c.abort = reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8);
  c.red = reinterpret_cast<float*>(smem + 2 * kMaxStages * 8 + 16);
  c.resid = reinterpret_cast<half*>(smem + kHeaderBytes);
  c.xin = reinterpret_cast<uint4*>(smem + kHeaderBytes + p.resid_bytes);
  c.xsum = reinterpret_cast<float*>(smem + kHeaderBytes + p.resid_bytes + p.xin_bytes);
  c.att = reinterpret_cast<float*>(smem + kHeaderBytes + p.resid_bytes + p.xin_bytes + p.xsum_bytes);
  c.part = reinterpret_cast<float*>(smem + kHeaderBytes + p.resid_bytes + p.xin_bytes + p.xsum_bytes + p.att_bytes);
  // the per-layer pointer table, copied once from global memory: every phase starts from these pointers, and a
  // global load in front of each would put an L2 round trip on the critical path ~10 times per layer
  StepLayer* lys = reinterpret_cast<StepLayer*>(smem + kHeaderBytes + p.resid_bytes + p.xin_bytes + p.xsum_bytes +
                                                p.att_bytes + p.part_bytes);
  c.ring = smem + kHeaderBytes + p.resid_bytes + p.xin_bytes + p.xsum_bytes + p.att_bytes + p.part_bytes + p.table_bytes;
  c.ctrl = p.ctrl;
  c.ns = p.ns;
  c.nopoll = p.debug & 1;
  c.stage_bytes = p.stage_bytes;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < p.ns; ++i) { mbar_init(&c.full[i], 1); mbar_init(&c.empty[i], kNCW); }
    *c.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The five matrix shapes of a step (qkv, o, gate|up, down, head) and this CTA's slice of each: computed once
  // (they involve integer divisions) and kept in shared memory for producer and consumers.
  Slice* sl = reinterpret_cast<Slice*>(smem + 512);
  if (tid < 5) {
    const int n_qkv_ = (p.n_q + 2 * p.n_kv) * p.D, n_att_ = p.n_q * p.D;
    const Mat shapes[5] = {{nullptr, n_qkv_, p.H, 0}, {nullptr, p.H, n_att_, 0}, {nullptr, p.I, p.H, 1},
                           {nullptr, p.H, p.I, 0}, {nullptr, p.V, p.H, 0}};
    sl[tid] = slice_of(shapes[tid], p.log2G, p.stage_w, blockIdx.x, gridDim.x);
  }
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.layers);
    uint4* dst = reinterpret_cast<uint4*>(lys);
    for (int i = tid; i < p.L * (int)(sizeof(StepLayer) / 16); i += kThreads) dst[i] = __ldg(src + i);
  }
  __syncthreads();
  const uint32_t epoch = ((volatile StepCtrl*)p.ctrl)->epoch + 1u;
  c.tagw = ((epoch % 65535u) + 1u) << 16;
  const int pos = p.pos[0];
  const int hpg = p.n_q / p.n_kv;

  const int n_qkv = (p.n_q + 2 * p.n_kv) * p.D, n_att = p.n_q * p.D;
  const int per_layer = n_qkv + n_att + p.H + p.I + p.H;   // exchange words per layer

  if (warp == kNCW) {
    // ================= producer =================
    RingPos rp = {0, 1u, 0};   // parity 1: the first pass over a fresh `empty` barrier does not wait
    for (int l = 0; l < p.L && !*c.abort; ++l) {
      const StepLayer& ly = lys[l];
      const Mat mats[4] = {{(const uint8_t*)ly.w[0], n_qkv, p.H, 0},
                           {(const uint8_t*)ly.w[1], p.H, n_att, 0},
                           {(const uint8_t*)ly.w[2], p.I, p.H, 1},
                           {(const uint8_t*)ly.w[3], p.H, p.I, 0}};
      produce(c, mats[0], sl[0], rp, lane);
      for (int h = cta; h < p.n_q && !*c.abort; h += ncta) produce_kv(c, p, ly, h / hpg, pos, rp, lane);
#pragma unroll
      for (int k = 1; k < 4; ++k)
        if (!*c.abort) produce(c, mats[k], sl[k], rp, lane);
    }
    if (!*c.abort) {
      const Mat head = {(const uint8_t*)p.w_head, p.V, p.H, 0};
      produce(c, head, sl[4], rp, lane);
    }
    // Leave only when every copy issued has landed. On the normal path the consumers have waited on every full
    // barrier already; on abort, wait (bounded) for the full barriers of the stages still in the ring.
    if (*c.abort) {
      const int it = rp.count;
      for (int k = max(0, it - c.ns); k < it; ++k) {
        const int slot = k % c.ns;
        for (int i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(&c.full[slot], (k / c.ns) & 1)) break;
      }
    }
    return;
  }

  // ================= consumers =================
  long long* tr = p.trace ? p.trace + (size_t)cta * (16 + 16 * p.L) : nullptr;
  int tri = 0;
#define TRACE()                                              \
  do {                                                       \
    if (tr && tid == 0) {                                    \
      long long t_;                                          \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); \
      tr[tri++] = t_;                                        \
    }                                                        \
  } while (0)
  TRACE();
  RingPos rp = {0, 0u, 0};
  // per-warp work split for the three row lengths (hidden, heads x head_dim, intermediate), in shared memory so
  // that picking one by phase does not cost registers
  WarpMap* wmaps = reinterpret_cast<WarpMap*>(smem + 640) + 3 * warp;
  if (lane < 3) wmaps[lane] = warp_map(lane == 0 ? p.H : (lane == 1 ? n_att : p.I), sl[lane == 0 ? 0 : (lane == 1 ? 1 : 3)].ups, warp);
  __syncwarp();
  unsigned long long best = 0ull;
  const half* emb_row = p.emb + (size_t)p.tok[0] * p.H;
  // RoPE factors and the page of this step's token depend only on pos: fetch them now, off the critical path
  float rope_c = 0.f, rope_s = 0.f;
  int page_new = 0;
  if (cta < p.n_q) {
    page_new = p.bt[pos >> p.log2P];
    if (tid < p.D) {
      rope_c = p.cos_t[(size_t)pos * (p.D >> 1) + tid % (p.D >> 1)];
      rope_s = p.sin_t[(size_t)pos * (p.D >> 1) + tid % (p.D >> 1)];
    }
  }
  // One loop body serves every GEMV of the step (4 per layer, then the LM head as "phase 0 of layer L"): the kernel
  // keeps a single copy of the staging, GEMV and attention code, which keeps the loop inside the instruction cache.
  const Mat head = {(const uint8_t*)p.w_head, p.V, p.H, 0};
#pragma unroll 1
  for (int step = 0; step <= 4 * p.L; ++step) {
    const int l = step >> 2, ph = step & 3;
    const bool is_head = l == p.L;
    const StepLayer& ly = lys[is_head ? 0 : l];
    uint32_t* E = p.xchg + (size_t)l * per_layer;
    uint32_t *Eqkv = E, *Eatt = E + n_qkv, *Eo = Eatt + n_att, *Eact = Eo + p.H, *Edown = Eact + p.I;
    Mat m;
    const uint32_t* Ein;
    const half* nw = nullptr;   // norm weight: non-null selects "residual add + RMSNorm" staging
    uint32_t* Eout;
    int out = OUT_TAGGED, n_in = p.H;
    if (ph == 0) {
      Ein = l == 0 ? nullptr : E - p.H;   // down of the previous layer: the last H words of its block
      nw = is_head ? p.norm_f : ly.ln1;
      m = is_head ? head : Mat{(const uint8_t*)ly.w[0], n_qkv, p.H, 0};
      Eout = Eqkv;
      out = is_head ? OUT_LOGITS : OUT_TAGGED;
    } else if (ph == 1) {
      Ein = Eatt; n_in = n_att;
      m = Mat{(const uint8_t*)ly.w[1], p.H, n_att, 0};
      Eout = Eo;
    } else if (ph == 2) {
      Ein = Eo; nw = ly.ln2;
      m = Mat{(const uint8_t*)ly.w[2], p.I, p.H, 1};
      Eout = Eact; out = OUT_SWIGLU;
    } else {
      Ein = Eact; n_in = p.I;
      m = Mat{(const uint8_t*)ly.w[3], p.H, p.I, 0};
      Eout = Edown;
    }
    const float resc = stage_x(c, Ein, emb_row, nw, n_in, p.eps, tid);
    TRACE();
    consume(c, m, sl[is_head ? 4 : ph], wmaps[ph == 1 ? 1 : (ph == 3 ? 2 : 0)], p.log2G, resc, rp, out, Eout, p.logits,
            best, tid);
    if (is_head) break;
    if (consumer_sync_or(*c.abort)) return;
    TRACE();
    if (ph == 0) {
      for (int h = cta; h < p.n_q; h += ncta) {
        attention_head<D>(c, p, ly, Eqkv, Eatt, h, pos, rope_c, rope_s, page_new, rp, tid);
        if (consumer_sync_or(*c.abort)) return;
      }
      TRACE();
    }
  }
  // this CTA's candidate: max over its threads' keys
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(c.att);
  {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
  }
  if (lane == 0) keys[warp] = best;
  if (consumer_sync_or(*c.abort)) return;
  TRACE();
  uint32_t* Earg = p.xchg + (size_t)p.L * per_layer;   // [ncta][4] words: idx low 16, idx high 16, value key, valid
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
      const uint2 v = poll4(c, Earg + 4 * k);
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
      TRACE();
    }
  }
#undef TRACE
}

size_t decode_step_smem_fixed(const StepParams& p) {
  return (size_t)kHeaderBytes + p.resid_bytes + p.xin_bytes + p.xsum_bytes + p.att_bytes + p.part_bytes + p.table_bytes;
}
int decode_step_threads() { return kThreads; }
int decode_step_max_stages() { return kMaxStages; }
int decode_step_consumer_warps() { return kNCW; }

cudaError_t decode_step_launch(const StepParams& p, int grid, size_t smem, cudaStream_t st) {
  static int configured_for = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_for != dev) {
    cudaError_t e = cudaFuncSetAttribute(decode_step_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_step_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
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
  return p.D == 64 ? cudaLaunchKernelEx(&cfg, decode_step_kernel<64>, p)
                   : cudaLaunchKernelEx(&cfg, decode_step_kernel<128>, p);
}

// ---- stream layout ----------------------------------------------------------------------------------------------------
// Rearranges one matrix (packed rows + scale/zero rows, the format of the quantizer) into the order the step kernel's
// producers read it: the slice of CTA 0 first, then CTA 1, ...; inside a slice one block per ring stage, made of the
// stage's packed rows followed by the same rows' (scale, zero) entries (gate|up: gate rows, up rows, gate sz, up sz).
// Every row contributes K/2 + 4 K/G bytes wherever it lands, so a stage's block starts at
// (index of its first row in slice order) * (K/2 + 4 K/G). One block per source row, one thread per 16-byte piece.
__global__ void repack_stream_kernel(const uint8_t* __restrict__ W, const uint8_t* __restrict__ SZ,
                                     uint8_t* __restrict__ out, int N, int K, int log2G, int gu, int ncta, int stage_w) {
  const int rb = K >> 1, sb = (K >> log2G) << 2, pieces = (rb + sb) >> 4;
  const int r = blockIdx.x;   // source row
  const Mat m = {nullptr, gu ? N / 2 : N, K, gu};
  const int units = gu ? m.N : (m.N + 1) >> 1;
  const int u = gu ? (r < m.N ? r : r - m.N) : r >> 1;
  const int base = units / ncta, rem = units % ncta, bnd = rem * (base + 1);
  const int cta = u < bnd ? u / (base + 1) : rem + (u - bnd) / max(base, 1);
  const Slice s = slice_of(m, log2G, stage_w, cta, ncta);
  const int st = (u - s.ub) / s.ups, u0 = s.ub + st * s.ups, u1 = min(s.ue, u0 + s.ups);
  const size_t rowall = (size_t)rb + sb;
  int slot, nrows;
  if (gu) { nrows = 2 * (u1 - u0); slot = (r < m.N ? 0 : u1 - u0) + (u - u0); }
  else { nrows = min(m.N, 2 * u1) - 2 * u0; slot = r - 2 * u0; }
  uint8_t* blk = out + (size_t)(2 * u0) * rowall;
  for (int i = threadIdx.x; i < pieces; i += blockDim.x) {
    const int off = i << 4;
    if (off < rb)
      *reinterpret_cast<uint4*>(blk + (size_t)slot * rb + off) = *reinterpret_cast<const uint4*>(W + (size_t)r * rb + off);
    else
      *reinterpret_cast<uint4*>(blk + (size_t)nrows * rb + (size_t)slot * sb + (off - rb)) =
          *reinterpret_cast<const uint4*>(SZ + (size_t)r * sb + (off - rb));
  }
}

cudaError_t repack_stream_dispatch(const void* W, const void* SZ, void* out, int N, int K, int log2G, int gu, int ncta,
                                   int stage_w, cudaStream_t st) {
  repack_stream_kernel<<<N, 128, 0, st>>>((const uint8_t*)W, (const uint8_t*)SZ, (uint8_t*)out, N, K, log2G, gu, ncta,
                                          stage_w);
  return cudaPeekAtLastError();
}

}  // namespace b200
