// One persistent kernel for the whole batch-1 decode step (all layers, LM head, greedy argmax).
//
// Why: at TinyLlama size the step streams 0.55 GB of INT4 weights, 86 us at the B200's measured HBM bandwidth,
// while the same step as 225 separate launches (the reference's structure, runtime/model.py:216-233) costs ~900 us
// of launch and pipeline-drain latency. Here one CTA per SM stays resident for the whole step:
//
//   * a producer warp streams this CTA's row tiles of every weight matrix - and, on the CTAs that do attention, the
//     K/V pages of their head - in the order the step consumes them, into a shared-memory ring with 1-D bulk async
//     copies (cp.async.bulk + mbarrier transaction counts). Neither weights nor cached K/V depend on this step's
//     activations, so the producer runs ahead of the computation by the depth of the ring and HBM never idles
//     while CTAs wait for each other;
//   * 11 consumer warps do the arithmetic out of the ring on the tensor cores (see "inner product" below), with the
//     row length K split across the warps: warp w owns the 128-column units w, w + 11, ... of every row tile, so it
//     needs only its own 128-element pieces of the activation vector and fetches exactly those - no CTA-wide staging
//     pass and no barrier in front of a GEMV. The warps' partial sums meet in shared memory once per matrix.
//     (Twelve warps in all, three per scheduler: a thread then has 168 registers, and this kernel must not spill -
//     with 227 KB of the SM's memory configured as shared there is next to no L1 left, so spilled registers would
//     be fetched from the L2, a microsecond each time, in a kernel whose phases last a microsecond. A thirteenth
//     warp puts four on one scheduler and caps every thread at 128 registers, seventeen warps at 96;)
//   * CTAs exchange activation vectors through global memory WITHOUT grid barriers: every fp16 result is stored
//     as a 32-bit word (tag << 16 | value) whose tag is this step's epoch; a consumer polls the words it needs until
//     all carry the current tag. One store + one load crosses the chip instead of fence + atomic + poll + load.
//     Every CTA keeps its own copy of the residual stream in shared memory (each warp its own units of it) and redoes
//     the (tiny) residual add and RMSNorm, so those never touch global memory.
//
// Weights are read from the tile layout of the tensor-core GEMV (gemv_tile_repack_kernel in gemv_w4a16.cu): per
// 16-row tile and 128-column unit one 1088-byte block, tiles back to back. A CTA owns a contiguous range of tiles of
// each matrix, so its share is one contiguous byte range and a ring stage is ONE bulk copy of up to `ups` blocks.
// The gate|up matrix uses the paired form of the layout (gate row i and up row i in one tile), which puts both
// halves of a SwiGLU output into the same thread.
//
// Inner product on the integer tensor cores. (word & 0x0F0F0F0F) and ((word >> 4) & 0x0F0F0F0F) are registers of four
// unsigned-byte weights each - three integer instructions for 8 weights - so a 16-row x 128-column block of W is
// four mma.m16n8k32 (u8 x s8 -> s32). The activations go in as 15-bit fixed point: staging scales a unit's x by
// 2^s (s from the unit's max|x|; a unit belongs to one warp, so this costs five shuffles and no reduction over the
// CTA), rounds to an integer X, |X| < 2^14, and splits it into two signed byte digits, X = 256 hi + lo. The digits
// ride in columns 0 and 1 of the B operand, which a batch-1 GEMV leaves idle anyway, the accumulation is exact, and
//     sum_k (q_k - z) * scale * x_k  =  scale * (2^-s * (256 C[.][0] + C[.][1]) - z * sum_k x_k)        per unit.
// Rounding x to 2^-14 of its unit's maximum is finer than the fp16 rounding x already carries, except for elements
// far below the maximum, whose absolute error it bounds by 2^-15 of the maximum (normwise ~1e-5 on the output).
// A NaN or infinity in a unit of x - which an integer cannot carry - turns that unit's factor 2^-s into NaN, so
// every row's output is NaN as in the reference.
// Why this form: a GEMV phase of this kernel is bound by instruction issue, and most instructions around the
// weights (LOP3, SHF, HFMA2) issue at half rate. Measured per tile-unit and warp, eight warps per SM: masked nibbles
// as fp16 subnormals into mma.m16n8k16, 5 integer instructions + 1 MMA per 8 weights of a row pair: 320 cycles; the
// same masks into half2 FMAs: 306; this form, 3 integer instructions per 8 weights and 4 MMAs per tile-unit: 195.
// (The e4m3 MMA of the same shape would fit too - a nibble in the low half of an e4m3 byte is exactly q * 2^-9 -
// but it is emulated on this part: 385.)
// The per-element weight this stands for is the format's dequantized weight (dequant_w4a16 in gemv_w4a16.cu proves
// the format bit-exactly).
//
// Phases per layer (the reference's operator order, with the same rounding points as its fused kernels):
//   A  resid += down[l-1] (layer 0: resid = embedding row);  x = RMSNorm(resid) * ln1;  qkv = Wqkv x
//   B  attention: query head h is shared by J CTAs (as many as the grid has to spare, at most 4), CTA h + j n_q
//      taking every J-th 128-token stage of the context: RoPE on q and k, (slice 0) append k, v to the paged cache,
//      then per-warp online softmax over the slice's cached tokens (from the ring), merged once across warps; the
//      slice's normalised output and log-sum-exp go to the exchange
//   C  o = Wo attn, attn merged from the J slices of each head while it is staged
//   D  resid += o;  x = RMSNorm(resid) * ln2;  act = SwiGLU(Wgate x, Wup x)
//   E  down = Wdown act
// then resid += down;  x = RMSNorm(resid) * norm_f;  logits = Whead x;  per-CTA argmax candidates; CTA 0 merges
// them (lowest index wins ties), writes tok, history[pos], pos + 1 and the new epoch.
// Barriers over the consumer threads per phase: one for sum(resid^2) where a norm precedes the GEMV, one between the
// warps' partial sums and the threads that add them up; the partial-sum buffer alternates between phases so that no
// third one is needed.
//
// Every wait (mbarrier or tag poll) is bounded. A wait that runs out records a code in StepCtrl::error, raises an
// abort flag that all later waits honour at once, and the CTA leaves after its copies in flight have landed; the
// host reads the code after the step. Nothing here can spin forever.
#include "common.cuh"
#include "decode_step.h"
#include <math_constants.h>

namespace b200 {

namespace {

#ifndef B200_STEP_CONSUMER_WARPS
#define B200_STEP_CONSUMER_WARPS 11   // build-time knob for measurements
#endif
constexpr int kNCW = B200_STEP_CONSUMER_WARPS;   // consumer warps (with the producer: 12 warps = 3 per scheduler, 168 registers)
constexpr int kNT = kNCW * 32;              // consumer threads
constexpr int kThreads = kNT + 32;          // + producer warp
constexpr int kMaxStages = 16;
constexpr int kSpinLimit = 1 << 18;         // polls / try_waits before a wait gives up (tens of milliseconds)
constexpr int kHeaderBytes = 2048;
constexpr int kMaxKvTokens = 128;           // cached tokens per ring stage in attention (3 rounds of 11 warps x 4 tokens)
constexpr int kKvRounds = (kMaxKvTokens + 4 * kNCW - 1) / (4 * kNCW);
constexpr int kSliceMinContext = 1152;      // cached tokens from which attention is cut into context slices
constexpr int kPollBatch = 4;               // exchange granules a lane keeps in flight while it polls (plain staging)
constexpr int kNormBatch = 2;               // the same where a norm follows: units of the residual stream per pass

enum : int { ERR_POLL = 1, ERR_FULL = 2, ERR_EMPTY = 3, ERR_TOKEN = 4 };

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

// ---- shared state of one CTA -----------------------------------------------------------------------------------
// Shared memory: [0, 128) full barriers, [128, 256) empty barriers, 256 abort flag, 272 sum scratch, 512 slices;
// from kHeaderBytes on: residual stream, then the areas whose offsets the host put into StepParams (off_*).
// Pointers into it are formed where they are used (one add of a kernel parameter) instead of being carried in
// registers through the whole step.
struct Cta {
  uint8_t* smem;
  const StepParams* p;   // the kernel's parameter block (constant bank)
  uint32_t tagw;         // (tag << 16)
#ifdef B200_STEP_TRACE
  long long* tr;         // this CTA's row of the trace array (thread 0 stamps), or null
#endif
  DEVI uint64_t* full(int i) const { return reinterpret_cast<uint64_t*>(smem) + i; }
  DEVI uint64_t* empty(int i) const { return reinterpret_cast<uint64_t*>(smem) + kMaxStages + i; }
  DEVI volatile int* abort() const { return reinterpret_cast<volatile int*>(smem + 2 * kMaxStages * 8); }
  // kNCW floats: the warps' shares of sum(resid^2)
  DEVI float* red() const { return reinterpret_cast<float*>(smem + 2 * kMaxStages * 8 + 16); }
  // [H] residual stream, private copy of the CTA; unit u belongs to warp u % kNCW
  DEVI half* resid() const { return reinterpret_cast<half*>(smem + kHeaderBytes); }
  // activations of the running GEMV as byte-digit B fragments, 256 bytes per unit; unit u is written and read by one warp only
  DEVI half* xin() const { return reinterpret_cast<half*>(smem + p->off_xin); }
  DEVI float* xsum() const { return reinterpret_cast<float*>(smem + p->off_xsum); }   // [Kmax / 128][2] sum, 2^-s
  DEVI float* att() const { return reinterpret_cast<float*>(smem + p->off_att); }     // attention scratch
  // partial dot products, [warp][row slot], two buffers used by alternate phases
  DEVI float* part() const { return reinterpret_cast<float*>(smem + p->off_part); }
  DEVI uint8_t* stage(int slot) const { return smem + p->off_ring + (size_t)slot * p->stage_bytes; }
  DEVI StepCtrl* ctrl() const { return p->ctrl; }
};

// Phase stamps of the instrumented build (-DB200_STEP_TRACE): thread 0 of the CTA stores the nanosecond timer at slot
// `at` of the CTA's trace row. The normal build compiles these calls to nothing.
#ifdef B200_STEP_TRACE
DEVI void stamp(const Cta& c, int at) {
  if (c.tr && threadIdx.x == 0) {
    long long t_;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));
    c.tr[at] = t_;
  }
}
#else
DEVI void stamp(const Cta&, int) {}
#endif
#ifdef B200_STEP_TRACE
DEVI long long now_ns() {
  long long t_;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));
  return t_;
}
// slot `at` <- a duration (ns) instead of a time
DEVI void stamp_value(const Cta& c, int at, long long v) {
  if (c.tr && threadIdx.x == 0) c.tr[at] = v;
}
#endif
constexpr int kTraceHead = 8, kTracePerPhase = 5, kTraceAttn = 5, kTracePerLayer = 4 * kTracePerPhase + kTraceAttn;

DEVI void raise(const Cta& c, int code) {
  if (!*c.abort()) {
    *c.abort() = 1;
    atomicCAS(&c.ctrl()->error, 0, code);
    c.ctrl()->abort = 1;
  }
}

// Wait for a ring barrier phase. Returns false (and raises) if the bound is hit or the step is already aborting.
// `nap` nanoseconds of sleep follow every failed attempt: a waiting warp must not eat the issue slots of the warps
// it shares a scheduler with (the producer waits for most of the step).
DEVI bool wait_bar(const Cta& c, uint64_t* bar, uint32_t parity, int code, unsigned nap = 0) {
#pragma unroll 1
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*c.abort()) return false;
    if (nap) __nanosleep(nap);
  }
  raise(c, code);
  return false;
}

// ---- tagged exchange words -----------------------------------------------------------------------------------------
// A word of step s carries tag (s mod 65535) + 1, so a word left over from step s - 65535 would pass for a fresh one.
// That cannot happen: every exchange word (every output row of every phase of every layer, and the argmax
// candidates) is rewritten in every step, so a word is never more than one step old when it is polled.
DEVI bool tags_ok(const Cta& c, uint4 v) {
  return ((((v.x ^ c.tagw) | (v.y ^ c.tagw) | (v.z ^ c.tagw) | (v.w ^ c.tagw)) >> 16) == 0);
}
DEVI uint2 payload(uint4 v) { return make_uint2((v.x & 0xFFFFu) | (v.y << 16), (v.z & 0xFFFFu) | (v.w << 16)); }

// Poll nb (<= NB, warp-uniform) granules of 4 tagged words, `stride` words apart, until all carry this
// step's tag; all loads of a round are in flight together. out[k] = the 4 fp16 payloads of granule k as 2 x half2.
template <int NB>
DEVI void poll_many(const Cta& c, const uint32_t* base, int stride, int nb, uint2 (&out)[NB]) {
  constexpr int kPollBatch = NB;
  uint4 v[kPollBatch];
#pragma unroll
  for (int k = 0; k < kPollBatch; ++k)
    if (k < nb) v[k] = ld_poll4(base + (size_t)k * stride);
  int spins = 0;
  for (;;) {
    bool ok = true;
#pragma unroll
    for (int k = 0; k < kPollBatch; ++k)
      if (k < nb && !tags_ok(c, v[k])) ok = false;
    if (ok || *c.abort()) break;
    if (++spins > kSpinLimit) { raise(c, ERR_POLL); break; }
    if ((spins & 255) == 0 && ((volatile StepCtrl*)c.ctrl())->abort) { *c.abort() = 1; break; }
#pragma unroll
    for (int k = 0; k < kPollBatch; ++k)
      if (k < nb && !tags_ok(c, v[k])) v[k] = ld_poll4(base + (size_t)k * stride);
  }
#pragma unroll
  for (int k = 0; k < kPollBatch; ++k)
    if (k < nb) out[k] = payload(v[k]);
}
DEVI uint2 poll4(const Cta& c, const uint32_t* p) {
  uint2 out[1];
  poll_many<1>(c, p, 0, 1, out);
  return out[0];
}
// The same for granules at unrelated places: entry k is at word offset off[k] from `base` (32-bit offsets: a dozen
// 64-bit pointers would not fit beside a dozen granules in flight); bit k of `mask` says whether entry k is in use
// (warp-uniform).
template <int NB>
DEVI void poll_list(const Cta& c, const uint32_t* base, const uint32_t (&off)[NB], uint32_t mask, uint2 (&out)[NB]) {
  uint4 v[NB];
#pragma unroll
  for (int k = 0; k < NB; ++k)
    if ((mask >> k) & 1u) v[k] = ld_poll4(base + off[k]);
  int spins = 0;
  for (;;) {
    bool ok = true;
#pragma unroll
    for (int k = 0; k < NB; ++k)
      if (((mask >> k) & 1u) && !tags_ok(c, v[k])) ok = false;
    if (ok || *c.abort()) break;
    if (++spins > kSpinLimit) { raise(c, ERR_POLL); break; }
    if ((spins & 255) == 0 && ((volatile StepCtrl*)c.ctrl())->abort) { *c.abort() = 1; break; }
#pragma unroll
    for (int k = 0; k < NB; ++k)
      if (((mask >> k) & 1u) && !tags_ok(c, v[k])) v[k] = ld_poll4(base + off[k]);
  }
#pragma unroll
  for (int k = 0; k < NB; ++k)
    if ((mask >> k) & 1u) out[k] = payload(v[k]);
}

// ---- x staging, per warp ------------------------------------------------------------------------------------------
// Warp w stages the units w, w + kNCW, ... of the activation vector: lane l holds granule l (4 values) of a unit.
// A unit's x goes to shared memory as the B fragments of the integer MMAs: X = round(x * 2^s), split into the signed
// byte digits hi and lo (X = 256 hi + lo, both in [-128, 127]), laid out as
//     xin words [unit][digit n = 0 (hi), 1 (lo)][t = 0..3][MMA m = 0..3][register r = 0..1]
// where lane (n, t) of tile_unit() loads its eight registers with two 16-byte reads. Register r of MMA m pairs with
// word 2 (m / 2) + r of the lane's four weight words, low nibbles (m even: elements e0 e4 e1 e5 of the word, in
// byte order) or high nibbles (m odd: e2 e6 e3 e7). Granule l = 4 elements of word (l % 8) / 2: elements e0..e3 on
// even lanes, e4..e7 on odd ones, so a lane pair swaps its packed bytes once and each lane permutes one register.
// xsum[2 u] = 2^-s sum X (for the zero-point term), xsum[2 u + 1] = 2^-s (both NaN if the unit is not finite).
DEVI void put_unit(const Cta& c, int u, uint2 v, int lane) {
  // max|x| of the unit from the bit patterns (the order of non-negative fp16 numbers is the order of their bits)
  const uint32_t m2 = __vmaxu2(v.x & 0x7FFF7FFFu, v.y & 0x7FFF7FFFu);
  const uint32_t mx = __reduce_max_sync(0xffffffffu, max(m2 & 0xFFFFu, m2 >> 16));
  const bool finite = mx < 0x7C00u;                       // no infinity, no NaN
  const int sh = 28 - max((int)(mx >> 10), 1);            // exponent field e: max|x| in [2^(e-15), 2^(e-14)) -> 2^sh max|x| in [2^13, 2^14)
  const float sc = __int_as_float((sh + 127) << 23);      // 2^sh, sh in [-2, 27]
  // round(x * 2^sh) + 128 in the low bits of a float: adding 1.5 * 2^23 + 128 rounds to an integer (nearest even)
  // and leaves it, in two's complement, in the mantissa. Byte 0 of that, with its top bit flipped, is the lo digit
  // (X & 255 read as a signed byte), byte 1 is the hi digit ((X + 128) >> 8).
  constexpr float kMagic = 12582912.f + 128.f;
  const float2 a = __half22float2(as_h2(v.x)), b = __half22float2(as_h2(v.y));
  const uint32_t w0 = __float_as_uint(fmaf(a.x, sc, kMagic)), w1 = __float_as_uint(fmaf(a.y, sc, kMagic));
  const uint32_t w2 = __float_as_uint(fmaf(b.x, sc, kMagic)), w3 = __float_as_uint(fmaf(b.y, sc, kMagic));
  const uint32_t kM = __float_as_uint(kMagic);            // w - kM = X
  const int xsum_i = __reduce_add_sync(0xffffffffu, (int)(w0 - kM) + (int)(w1 - kM) + (int)(w2 - kM) + (int)(w3 - kM));
  const float resc = finite ? __int_as_float((127 - sh) << 23) : __int_as_float(0x7fc00000);   // 2^-sh, or NaN
  if (lane == 0) {
    c.xsum()[2 * u] = (float)xsum_i * resc;               // the sum of what the MMAs multiply, rescaled
    c.xsum()[2 * u + 1] = resc;
  }
  // bytes: this granule's 4 elements in order
  const uint32_t lo = __byte_perm(__byte_perm(w0, w1, 0x0040), __byte_perm(w2, w3, 0x0040), 0x5410) ^ 0x80808080u;
  const uint32_t hi = __byte_perm(__byte_perm(w0, w1, 0x0051), __byte_perm(w2, w3, 0x0051), 0x5410);
  const int t = lane >> 3, wd = (lane & 7) >> 1, odd = lane & 1;
  uint32_t* dst = reinterpret_cast<uint32_t*>(c.xin()) + (size_t)u * 64 + t * 8 + ((wd >> 1) * 2 + odd) * 2 + (wd & 1);
  const uint32_t hi_o = __shfl_xor_sync(0xffffffffu, hi, 1), lo_o = __shfl_xor_sync(0xffffffffu, lo, 1);
  // even lane (e0..e3; partner e4..e7): low-nibble register (e0 e4 e1 e5); odd lane: high-nibble one (e2 e6 e3 e7)
  dst[0] = odd ? __byte_perm(hi, hi_o, 0x3726) : __byte_perm(hi, hi_o, 0x5140);
  dst[32] = odd ? __byte_perm(lo, lo_o, 0x3726) : __byte_perm(lo, lo_o, 0x5140);
}

// x <- E[0..K) (tagged).
DEVI void stage_plain(const Cta& c, const uint32_t* E, int K, int warp, int lane) {
  const int nunit = K >> 7;
  for (int u0 = warp; u0 < nunit; u0 += kNCW * kPollBatch) {
    const int nb = min(kPollBatch, (nunit - u0 + kNCW - 1) / kNCW);
    uint2 v[kPollBatch];
    poll_many(c, E + 128 * u0 + 4 * lane, 128 * kNCW, nb, v);
#pragma unroll
    for (int k = 0; k < kPollBatch; ++k)
      if (k < nb) put_unit(c, u0 + kNCW * k, v[k], lane);
  }
  __syncwarp();
}

// x <- the attention output, merged from the J context slices of every head while it is staged: slice j of head h
// left its normalised output o_j (Eatt + j n_att) and its log-sum-exp l_j as two fp16 words, value and remainder
// (Else + h * step_lse_words(J) + 2 j); x = sum_j e^(l_j - max l) o_j / sum_j e^(l_j - max l). A slice that saw no
// token has l_j = -inf and o_j = 0. Lane l of the warp that owns unit u holds 4 values of one head.
// A function of its own, called (with the CTA's state by value, in registers) only in steps with a sliced context:
// inlined into the one loop body that serves every phase of the step it made the GEMV phases of EVERY step a fifth
// slower (measured; what the compiler does with that loop depends on everything in it - moving put_unit out of line,
// which shrinks the body by 12 KB, costs 6 %, and so does doing two tiles at once in gemv()).
__device__ __noinline__ void stage_attn(const Cta c, const uint32_t* Eatt, const uint32_t* Else, int J, int n_att, int D, int warp,
                     int lane) {
  constexpr int NL = (kStepMaxAttSlices + 1) / 2;   // granules of log-sum-exp words per head
  const int nunit = n_att >> 7, lsew = step_lse_words(J), ng = lsew >> 2;
  const uint32_t lbase = (uint32_t)(Else - Eatt);
  for (int u = warp; u < nunit; u += kNCW) {
    const int i = 128 * u + 4 * lane, h = i / D;
    // While the slices are still at work the warp polls the log-sum-exp words only: one or two addresses per head,
    // the same for all lanes of a head, instead of J granules per lane - 148 CTAs polling every partial would keep
    // the L2 busy with nothing else. When those are there the outputs are too, or nearly (the second poll checks
    // their tags all the same). One unit at a time: more granules in flight would not fit into the registers, and
    // this kernel must not spill.
    uint32_t loff[NL], ooff[kStepMaxAttSlices];   // word offsets from Eatt (Else lies behind it)
#pragma unroll
    for (int g = 0; g < NL; ++g) loff[g] = lbase + (uint32_t)(h * lsew + 4 * g);
#pragma unroll
    for (int k = 0; k < kStepMaxAttSlices; ++k) ooff[k] = (uint32_t)(k * n_att + i);
    uint2 lv[NL], v[kStepMaxAttSlices];
    poll_list(c, Eatt, loff, (1u << ng) - 1u, lv);
    poll_list(c, Eatt, ooff, (1u << J) - 1u, v);
    float lse[kStepMaxAttSlices], M = -CUDART_INF_F;
#pragma unroll
    for (int k = 0; k < kStepMaxAttSlices; ++k) {
      lse[k] = -CUDART_INF_F;
      if (k < J) {
        const uint2 pr = lv[k >> 1];
        const float2 f = __half22float2(as_h2((k & 1) ? pr.y : pr.x));   // (value, remainder)
        lse[k] = f.x + f.y;
        M = fmaxf(M, lse[k]);
      }
    }
    float W = 0.f, o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
    for (int k = 0; k < kStepMaxAttSlices; ++k) {
      if (k < J) {
        const float w = __expf(lse[k] - M);   // the slice with the step's own token is never empty: M is finite
        const float2 x01 = __half22float2(as_h2(v[k].x)), x23 = __half22float2(as_h2(v[k].y));
        W += w;
        o0 = fmaf(w, x01.x, o0), o1 = fmaf(w, x01.y, o1), o2 = fmaf(w, x23.x, o2), o3 = fmaf(w, x23.y, o3);
      }
    }
    const float rW = 1.f / W;
    uint2 o;
    o.x = as_u32(__floats2half2_rn(o0 * rW, o1 * rW));
    o.y = as_u32(__floats2half2_rn(o2 * rW, o3 * rW));
    put_unit(c, u, o, lane);
  }
  __syncwarp();
}

// resid <- resid + delta (delta tagged; or resid <- emb row when E == nullptr), then
// x <- w * half(float(resid) * rsqrt(mean(resid^2) + eps)).  One barrier over the consumer threads (the sum).
DEVI void stage_norm(const Cta& c, const uint32_t* E, const half* emb_row, const half* w, int H, float eps, int warp,
                     int lane) {
  const int nunit = H >> 7;
  uint2* rs = reinterpret_cast<uint2*>(c.resid());
  const uint2* wg = reinterpret_cast<const uint2*>(w);
  // the norm weights of the first batch are requested before the poll: their latency hides behind the wait
  uint2 wv0[kNormBatch];
#pragma unroll
  for (int k = 0; k < kNormBatch; ++k)
    if (warp + kNCW * k < nunit) wv0[k] = __ldg(wg + 32 * (warp + kNCW * k) + lane);
  float ss = 0.f;
  for (int u0 = warp; u0 < nunit; u0 += kNCW * kNormBatch) {
    const int nb = min(kNormBatch, (nunit - u0 + kNCW - 1) / kNCW);
    uint2 d[kNormBatch];
    if (E) poll_many(c, E + 128 * u0 + 4 * lane, 128 * kNCW, nb, d);
#pragma unroll
    for (int k = 0; k < kNormBatch; ++k) {
      if (k < nb) {
        const int idx = 32 * (u0 + kNCW * k) + lane;
        uint2 r;
        if (E) {
          r = rs[idx];
          r.x = as_u32(__hadd2(as_h2(r.x), as_h2(d[k].x)));
          r.y = as_u32(__hadd2(as_h2(r.y), as_h2(d[k].y)));
        } else {
          r = __ldg(reinterpret_cast<const uint2*>(emb_row) + idx);
        }
        rs[idx] = r;
        const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
        ss = fmaf(a.x, a.x, fmaf(a.y, a.y, fmaf(b.x, b.x, fmaf(b.y, b.y, ss))));
      }
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) c.red()[warp] = ss;
  consumer_sync();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < kNCW; ++k) tot += c.red()[k];
  const float rinv = rsqrtf(tot / (float)H + eps);
  int j = 0;
  for (int u = warp; u < nunit; u += kNCW, ++j) {
    const int idx = 32 * u + lane;
    const uint2 r = rs[idx];   // this lane's own write
    uint2 wv;
    if (j < kNormBatch) {
      wv = wv0[0];
#pragma unroll
      for (int k = 1; k < kNormBatch; ++k)
        if (j == k) wv = wv0[k];
    } else {
      wv = __ldg(wg + idx);
    }
    const float2 a = __half22float2(as_h2(r.x)), b = __half22float2(as_h2(r.y));
    uint2 o;
    o.x = as_u32(__hmul2(as_h2(wv.x), __floats2half2_rn(a.x * rinv, a.y * rinv)));
    o.y = as_u32(__hmul2(as_h2(wv.y), __floats2half2_rn(b.x * rinv, b.y * rinv)));
    put_unit(c, u, o, lane);
  }
  __syncwarp();
}

// ---- GEMV phase -----------------------------------------------------------------------------------------------------
// A weight matrix in tile layout. N = outputs (for gate|up: I, each output made of a gate and an up row).
struct Mat {
  const uint8_t* base;
  int N, K;
  int paired;          // 1: gate|up tiles (8 gate rows + their 8 up rows)
};

struct Slice { int t0, nt; };   // this CTA's tiles [t0, t0 + nt) of a matrix

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

// Whole tiles are dealt to the CTAs as evenly as they go: a GEMV phase of the step is a handful of tile-units per
// warp, so one tile more or less on a CTA moves the phase by a tenth of a microsecond, and no row of padding is
// ever streamed.
DEVI Slice slice_of(int rows, int paired, int cta, int ncta) {
  const int tiles = paired ? (rows + 7) >> 3 : (rows + 15) >> 4;
  const int base = tiles / ncta, rem = tiles % ncta;
  Slice s;
  s.t0 = cta * base + min(cta, rem);
  s.nt = base + (cta < rem ? 1 : 0);
  return s;
}

// Producer: issue every stage of one matrix slice, one copy each (a bulk copy costs ~0.2 us to issue whatever its
// size, so several small copies per stage would make the producer the bottleneck).
DEVI void produce(const Cta& c, const Mat& m, const Slice& s, RingPos& rp, int lane) {
  const int nunit = m.K >> 7, NU = s.nt * nunit;
  const uint8_t* src = m.base + (size_t)s.t0 * nunit * kTileUnitBytes;
  for (int i0 = 0; i0 < NU; i0 += c.p->ups, advance(rp, c.p->ns)) {
    const int slot = rp.slot;
    if (!wait_bar(c, c.empty(slot), rp.parity, ERR_EMPTY, 200)) return;
    if (lane == 0) {
      const uint32_t bytes = (uint32_t)(min(c.p->ups, NU - i0) * kTileUnitBytes);
      mbar_expect_tx(c.full(slot), bytes);
      bulk_g2s(c.stage(slot), src + (size_t)i0 * kTileUnitBytes, bytes, c.full(slot));
    }
  }
}

// Cached tokens per attention ring stage: K rows in the first half of the stage, V rows in the second.
DEVI int kv_tokens_per_stage(const StepParams& p) {
  int t = min(kMaxKvTokens, p.stage_w / (4 * p.D));
  return t & ~((1 << p.log2P) - 1);
}

// Producer: the cached K/V rows [0, pos) of one kv head, page by page, for context slice j of J: the stages j, j + J,
// ... of the context. Whole pages are copied; rows at or beyond pos in the last page are ignored by the consumer.
DEVI void produce_kv(const Cta& c, const StepParams& p, const StepLayer& ly, int kvh, int j, int J, int pos, RingPos& rp,
                     int lane) {
  const int tps = kv_tokens_per_stage(p), pps = tps >> p.log2P;
  const uint32_t page_bytes = (uint32_t)(p.D * 2) << p.log2P;
  const int nst = (pos + tps - 1) / tps;
  for (int st = j; st < nst; st += J, advance(rp, c.p->ns)) {
    const int slot = rp.slot;
    if (!wait_bar(c, c.empty(slot), rp.parity, ERR_EMPTY, 200)) return;
    const int pg0 = st * pps, npg = min(pps, ((pos + (1 << p.log2P) - 1) >> p.log2P) - pg0);
    uint8_t* dst = c.stage(slot);
    if (lane == 0) mbar_expect_tx(c.full(slot), 2 * npg * page_bytes);
    __syncwarp();
    for (int pg = lane; pg < npg; pg += 32) {
      const size_t off = ((size_t)p.bt[pg0 + pg] * p.n_kv + kvh) * page_bytes;
      bulk_g2s(dst + pg * page_bytes, reinterpret_cast<const uint8_t*>(ly.kc) + off, page_bytes, c.full(slot));
      bulk_g2s(dst + (size_t)tps * p.D * 2 + pg * page_bytes, reinterpret_cast<const uint8_t*>(ly.vc) + off,
               page_bytes, c.full(slot));
    }
  }
}

// One tile-unit block (at `tu` in the ring) against unit u of x: the dot products of row slots g (ya) and g + 8 (yb)
// over the unit's 128 columns, scaled and with the zero-point term; meaningful on lanes t == 0.
// Lane (g, t) reads 16 bytes of row slot g and of row slot g + 8 (columns 32 t .. 32 t + 31 of the unit); lanes
// (0, t) carry the hi digits of the matching 32 activations as the B operand, lanes (1, t) the lo digits, the other
// lanes zeros. Four MMAs in two independent chains.
DEVI void tile_unit(const Cta& c, const uint8_t* tu, int u, int lane, float& ya, float& yb) {
  const int g = lane >> 2, t = lane & 3;
  uint4 x0 = make_uint4(0u, 0u, 0u, 0u), x1 = x0;
  if (g < 2) {
    const uint4* xp = reinterpret_cast<const uint4*>(c.xin()) + (size_t)u * 16 + (g * 4 + t) * 2;
    x0 = xp[0];   // MMAs 0, 1: registers (m0 r0, m0 r1, m1 r0, m1 r1)
    x1 = xp[1];   // MMAs 2, 3
  }
  const uint4 wa = *reinterpret_cast<const uint4*>(tu + 16 * lane);
  const uint4 wb = *reinterpret_cast<const uint4*>(tu + 512 + 16 * lane);
  constexpr uint32_t kNib = 0x0F0F0F0Fu;
  int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0};
  mma16832_u8s8(c0, wa.x & kNib, wb.x & kNib, wa.y & kNib, wb.y & kNib, x0.x, x0.y);
  mma16832_u8s8(c1, (wa.x >> 4) & kNib, (wb.x >> 4) & kNib, (wa.y >> 4) & kNib, (wb.y >> 4) & kNib, x0.z, x0.w);
  mma16832_u8s8(c0, wa.z & kNib, wb.z & kNib, wa.w & kNib, wb.w & kNib, x1.x, x1.y);
  mma16832_u8s8(c1, (wa.z >> 4) & kNib, (wb.z >> 4) & kNib, (wa.w >> 4) & kNib, (wb.w >> 4) & kNib, x1.z, x1.w);
  // lanes t == 0: C columns 0 (hi digits) and 1 (lo digits) of rows g (c[0], c[1]) and g + 8 (c[2], c[3])
  const float2 sa = __half22float2(*reinterpret_cast<const half2*>(tu + 1024 + 4 * g));
  const float2 sc = __half22float2(*reinterpret_cast<const half2*>(tu + 1024 + 4 * (g + 8)));
  const float xs = c.xsum()[2 * u], resc = c.xsum()[2 * u + 1];
  const float va = (float)(((c0[0] + c1[0]) << 8) + (c0[1] + c1[1]));
  const float vb = (float)(((c0[2] + c1[2]) << 8) + (c0[3] + c1[3]));
  ya = fmaf(sa.x, fmaf(va, resc, -sa.y * xs), ya);
  yb = fmaf(sc.x, fmaf(vb, resc, -sc.y * xs), yb);
}

// Consumer side of one matrix slice, one warp's share. The slice is the sequence of tile-unit blocks
// (tile 0 unit 0, tile 0 unit 1, ..., tile 1 unit 0, ...), `ups` of them per ring stage; warp w takes the blocks of
// units w, w + kNCW, ... of every tile, two at a time where the ring stage holds both (two independent instruction
// streams for the scheduler to interleave). The activations are re-read from shared memory for every block: keeping
// them in registers across tiles was measured and loses - it pushes the kernel over its registers, and a spilled
// register costs an L2 round trip here. Doing two tiles of a stage together (four independent blocks) was measured
// too and loses 3 %. When the warp has passed its last unit of a tile, lanes t == 0 leave the
// two partial sums of rows g and g + 8 in part[warp][16 * tile + row slot]. A warp whose units do not exist
// (K < 1024) only keeps the ring's barriers moving.
DEVI void gemv(const Cta& c, const Mat& m, const Slice& s, float* part, int pstride, RingPos& rp, int warp, int lane,
               int trace_at) {
  const int g = lane >> 2, t = lane & 3;
  const int nunit = m.K >> 7, NU = s.nt * nunit;
  const bool active = warp < nunit;
  int tl = 0, u = warp, idx = warp;   // the warp's next block: local tile, unit, place in the sequence
  float ya = 0.f, yb = 0.f;
#ifdef B200_STEP_TRACE
  long long waited = 0;
#endif
  for (int i0 = 0; i0 < NU; i0 += c.p->ups, advance(rp, c.p->ns)) {
    const int slot = rp.slot;
#ifdef B200_STEP_TRACE
    const long long w0 = now_ns();
#endif
    const bool ok = wait_bar(c, c.full(slot), rp.parity, ERR_FULL);
#ifdef B200_STEP_TRACE
    waited += now_ns() - w0;   // time this warp spent waiting for ring stages of the matrix
#endif
    const int end = min(NU, i0 + c.p->ups);
    const uint8_t* sb = c.stage(slot) - (size_t)i0 * kTileUnitBytes;   // block idx of the sequence is at sb + idx * 1088
    if (ok && active) {
      while (idx < end) {
        const bool two = u + kNCW < nunit && idx + kNCW < end;   // the next unit of the same tile is in this stage too
        float ya2 = 0.f, yb2 = 0.f;
        tile_unit(c, sb + (size_t)idx * kTileUnitBytes, u, lane, ya, yb);
        if (two) tile_unit(c, sb + (size_t)(idx + kNCW) * kTileUnitBytes, u + kNCW, lane, ya2, yb2);
        ya += ya2;
        yb += yb2;
        const int step = two ? 2 * kNCW : kNCW;
        u += step;
        if (u >= nunit) {
          if (t == 0) {
            part[warp * pstride + 16 * tl + g] = ya;
            part[warp * pstride + 16 * tl + g + 8] = yb;
          }
          ya = yb = 0.f;
          ++tl;
          u = warp;
          idx = tl * nunit + warp;
        } else {
          idx += step;
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(c.empty(slot));
  }
#ifdef B200_STEP_TRACE
  stamp_value(c, trace_at, waited);
#endif
}

enum : int { OUT_TAGGED = 0, OUT_SWIGLU = 1, OUT_LOGITS = 2 };

// Sum of one row slot over the nwa warps that hold a share of it, always in the same order. With all warps (rows of
// 1024 weights and more) the loads are issued together and added as a tree: the loop form would make every load
// wait for the add before it.
DEVI float sum_partials(const float* p, int pstride, int nwa) {
  if (nwa == kNCW) {
    float v[kNCW];
#pragma unroll
    for (int k = 0; k < kNCW; ++k) v[k] = p[k * pstride];
#pragma unroll
    for (int k = 0; k + 1 < kNCW; k += 2) v[k] += v[k + 1];     // pairs, then the pair sums in order
    float y = v[0];
#pragma unroll
    for (int k = 2; k < kNCW; k += 2) y += v[k];
    return y;
  }
  float y = 0.f;
  for (int k = 0; k < nwa; ++k) y += p[k * pstride];
  return y;
}

// After the barrier that follows gemv(): thread i adds the warps' partial sums of row slot i in a fixed order
// (deterministic) and emits the output.
//   OUT_TAGGED: E[row] <- tagged y.  OUT_SWIGLU: E[i] <- tagged half(silu(gate_i)) * up_i.
//   OUT_LOGITS: logits[row] <- y, and `best` tracks this thread's maximum.
DEVI void reduce_emit(const Cta& c, const Mat& m, const Slice& s, const float* part, int pstride, const int OUT,
                      uint32_t* E, half* logits, unsigned long long& best, int tid) {
  const int nwa = min(kNCW, m.K >> 7);
  if (OUT == OUT_SWIGLU) {
    for (int i = tid; i < 8 * s.nt; i += kNT) {
      const int slot = 16 * (i >> 3) + (i & 7), o = 8 * s.t0 + i;
      if (o >= m.N) continue;
      const float ga = sum_partials(part + slot, pstride, nwa), up = sum_partials(part + slot + 8, pstride, nwa);
      const half h0 = __float2half(ga), h1 = __float2half(up);
      const float gf = __half2float(h0);
      const half sl = __float2half(__fdividef(gf, 1.f + __expf(-gf)));
      st_tagged(E + o, c.tagw | (uint32_t)__half_as_ushort(__hmul(sl, h1)));
    }
    return;
  }
  for (int i = tid; i < 16 * s.nt; i += kNT) {
    const int row = 16 * s.t0 + i;
    if (row >= m.N) continue;
    const half h = __float2half(sum_partials(part + i, pstride, nwa));
    if (OUT == OUT_TAGGED) {
      st_tagged(E + row, c.tagw | (uint32_t)__half_as_ushort(h));
    } else {
      logits[row] = h;
      if (!__hisnan(h)) { const unsigned long long key = argmax_key(h, row); best = key > best ? key : best; }
    }
  }
}

// ---- attention for one query head, one context slice ------------------------------------------------------------------
// All consumer threads of the CTA. q, k, v of this step come from the tagged qkv exchange, the cached tokens of slice
// j (ring stages j, j + J, ... of the context) from ring stages filled by produce_kv; slice 0 also takes the token
// of this step and writes it to the cache. Lane (t = lane >> 3, c = lane & 7) of warp w owns token slot 4 w + t of a
// stage and dims [c D/8, (c+1) D/8) of it; each warp keeps a private online-softmax state, merged once at the end.
// Output: the slice's normalised partial at Eattn + j n_att and its log-sum-exp at Else (see stage_attn).
template <int D>
DEVI void attention_head(const Cta& c, const StepParams& p, const StepLayer& ly, uint32_t* E, int u, int pos,
                         RingPos& rp, int tid, int trace_at) {
  // E: the layer's exchange block; u: attention unit = head u % n_q, slice u / n_q. Whatever the publishing code at
  // the end needs is recomputed there from u and the parameter block: the fold loop in between is where this kernel's
  // register pressure peaks, and every value carried across it costs a register there.
  constexpr int D2 = D / 2, G4 = D / 4, DPL = D / 8;
  const int warp = tid >> 5, lane = tid & 31, ts = lane >> 3, ch = lane & 7;
  const int J = p.att_slices, h = u % p.n_q, j = u / p.n_q;
  const int Js = pos >= kSliceMinContext ? J : 1;            // stride of a slice's stages: 1 = slice 0 takes them all
  const int hpg = p.n_q / p.n_kv, kvh = h / hpg;
  const int tps = kv_tokens_per_stage(p);
  const int nst = (pos + tps - 1) / tps;                       // stages of the whole context
  const uint32_t* Eqkv = E;
  if (j > 0 && (j >= nst || Js == 1)) {
    // no cached token falls into this slice: an empty partial, without touching q, k, v or the ring
    uint32_t* Eo = E + (size_t)(p.n_q + 2 * p.n_kv) * D + (size_t)j * p.n_q * D + (size_t)h * D;
    uint32_t* El = E + (size_t)(p.n_q + 2 * p.n_kv) * D + (size_t)J * p.n_q * D + (size_t)h * step_lse_words(J) + 2 * j;
    const uint32_t ninf = c.tagw | 0xFC00u;                    // fp16 -inf
    if (tid < D) st_tagged(Eo + tid, c.tagw);
    if (tid == 0) {
      st_tagged(El, ninf);
      st_tagged(El + 1, c.tagw);
      if ((J & 1) && j == J - 1) { st_tagged(El + 2, ninf); st_tagged(El + 3, c.tagw); }
    }
    return;
  }
  float* qf = c.att();                                         // [D] rotated q * 1/sqrt(D)
  half* knew = reinterpret_cast<half*>(c.att() + D);           // [D] rotated k of this step
  half* vnew = knew + D;                                     // [D]
  half* raw = vnew + D;                                      // [3 D] un-rotated q, k, v
  float* wo = c.att() + 4 * D;                                 // [kNCW][D] per-warp outputs
  float* wm = wo + kNCW * D;                                 // [kNCW] per-warp max
  float* wl = wm + kNCW;                                     // [kNCW] per-warp sum
  const float* rope = wl + kNCW;                             // [D/2] cos, [D/2] sin, then the page of this step's token
  const int pmask = (1 << p.log2P) - 1;

  if (tid < 3 * G4) {
    const int which = tid / G4, g = tid % G4;
    const int head = which == 0 ? h : (which == 1 ? p.n_q + kvh : p.n_q + p.n_kv + kvh);
    reinterpret_cast<uint2*>(raw)[tid] = poll4(c, Eqkv + (size_t)head * D + 4 * g);
  }
  consumer_sync();
  if (tid < 2 * D) {
    const int slot_new = pos & pmask;
    const int page_new = reinterpret_cast<const int*>(rope)[D];
    const float cs = rope[tid % D2], sn = rope[D2 + tid % D2];
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
        if (h % hpg == 0 && j == 0) { ly.kc[row_new + i] = ra; ly.kc[row_new + i + D2] = rb; }
      }
    } else {
      const int i = tid - D;
      const half v = raw[2 * D + i];
      vnew[i] = v;
      if (h % hpg == 0 && j == 0) ly.vc[row_new + i] = v;
    }
  }
  consumer_sync();

  stamp(c, trace_at);
  float qreg[DPL];
#pragma unroll
  for (int d = 0; d < DPL; ++d) qreg[d] = qf[ch * DPL + d];
  float m = -CUDART_INF_F, l = 0.f, acc[DPL];
#pragma unroll
  for (int d = 0; d < DPL; ++d) acc[d] = 0.f;

  // Fold kKvRounds rounds of 4 tokens per warp into the warp's online-softmax state. Round r, token slot ts: the K row
  // at byte koff[r] of shared memory, the V row at voff[r], counted if valid[r] (a slot that is not valid reads this
  // step's own k, v - real data, masked by its score; stale bytes of the ring could be NaN patterns, and 0 * NaN
  // would poison the sum). The scores of all rounds are computed independently and share ONE max / rescale step, so
  // a ring stage costs one dependent chain (loads, dot product, shuffles, exponentials, accumulate) whatever its
  // token count; the round count is fixed so that the chain carries no predicates.
  auto fold = [&](const uint32_t (&koff)[kKvRounds], const uint32_t (&voff)[kKvRounds], const bool (&valid)[kKvRounds]) {
    float s[kKvRounds];
#pragma unroll
    for (int r = 0; r < kKvRounds; ++r) {
      const half* kp = reinterpret_cast<const half*>(c.smem + koff[r]);
      float kf[DPL], a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int d8 = 0; d8 < DPL; d8 += 8) unpack8(*reinterpret_cast<const uint4*>(kp + d8), kf + d8);
#pragma unroll
      for (int d = 0; d < DPL; d += 2) { a0 = fmaf(kf[d], qreg[d], a0); a1 = fmaf(kf[d + 1], qreg[d + 1], a1); }
      float a = a0 + a1;
      a += __shfl_xor_sync(0xffffffffu, a, 1);
      a += __shfl_xor_sync(0xffffffffu, a, 2);
      a += __shfl_xor_sync(0xffffffffu, a, 4);
      s[r] = valid[r] ? a : -CUDART_INF_F;
    }
    float mw = s[0];
#pragma unroll
    for (int r = 1; r < kKvRounds; ++r) mw = fmaxf(mw, s[r]);
    mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 8));
    mw = fmaxf(mw, __shfl_xor_sync(0xffffffffu, mw, 16));
    const float mn = fmaxf(m, mw);
    if (mn == -CUDART_INF_F) return;           // nothing valid yet in this warp (warp-uniform)
    const float alpha = __expf(m - mn);
    m = mn;
    l *= alpha;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[d] *= alpha;
#pragma unroll
    for (int r = 0; r < kKvRounds; ++r) {
      const half* vp = reinterpret_cast<const half*>(c.smem + voff[r]);
      const float pr = __expf(s[r] - mn);      // a masked slot: e^(-inf) = 0
      l += pr;
      float vf[DPL];
#pragma unroll
      for (int d8 = 0; d8 < DPL; d8 += 8) unpack8(*reinterpret_cast<const uint4*>(vp + d8), vf + d8);
#pragma unroll
      for (int d = 0; d < DPL; ++d) acc[d] = fmaf(pr, vf[d], acc[d]);
    }
  };

  // The cached tokens come stage by stage from the ring. The token of this step (rotated k, v in the attention
  // scratch) belongs to slice 0 and rides along as token number nt of that slice's last stage: a stage holds at most
  // kMaxKvTokens tokens and the warps' slots cover 4 kNCW kKvRounds > kMaxKvTokens, so there is always a slot for it
  // and it costs no chain of its own.
  static_assert(4 * kNCW * kKvRounds > kMaxKvTokens, "a stage needs a spare slot for the token of this step");
  const bool takes_new = j == 0;
  const uint32_t knew_off = (uint32_t)(reinterpret_cast<const uint8_t*>(knew) - c.smem) + ch * DPL * 2;
  const uint32_t vnew_off = (uint32_t)(reinterpret_cast<const uint8_t*>(vnew) - c.smem) + ch * DPL * 2;
#ifdef B200_STEP_TRACE
  long long waited = 0;
#endif
  for (int st = j; st < nst || (nst == 0 && st == 0); st += Js) {  // nst == 0 (empty cache, slice 0): one pass
    const bool have = st < nst, last = st + Js >= nst;              // without a ring stage
    const int slot = rp.slot;
#ifdef B200_STEP_TRACE
    const long long w0 = now_ns();
#endif
    const bool ok = have ? wait_bar(c, c.full(slot), rp.parity, ERR_FULL) : true;
#ifdef B200_STEP_TRACE
    waited += now_ns() - w0;
#endif
    const uint32_t kbase = c.p->off_ring + (uint32_t)slot * c.p->stage_bytes + ch * DPL * 2;
    const uint32_t vbase = kbase + (uint32_t)tps * D * 2;
    const int nt = have ? min(tps, pos - st * tps) : 0;
    if (ok) {
      uint32_t koff[kKvRounds], voff[kKvRounds];
      bool valid[kKvRounds];
#pragma unroll
      for (int r = 0; r < kKvRounds; ++r) {
        const int jt = 4 * warp + ts + 4 * kNCW * r;   // token slot of the stage
        valid[r] = jt < nt || (takes_new && last && jt == nt);
        koff[r] = jt < nt ? kbase + (uint32_t)jt * (D * 2) : knew_off;
        voff[r] = jt < nt ? vbase + (uint32_t)jt * (D * 2) : vnew_off;
      }
      fold(koff, voff, valid);
    }
    if (have) {
      __syncwarp();
      if (lane == 0) mbar_arrive(c.empty(slot));
      advance(rp, c.p->ns);
    }
  }
  stamp(c, trace_at + 1);
#ifdef B200_STEP_TRACE
  stamp_value(c, trace_at + 4, waited);   // a duration: what warp 0 waited for the K/V stages
#endif

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
    const int Jp = p.att_slices, hp = u % p.n_q, jp = u / p.n_q;
    uint32_t* Eo = E + (size_t)(p.n_q + 2 * p.n_kv) * D + (size_t)jp * p.n_q * D + (size_t)hp * D;
    uint32_t* El = E + (size_t)(p.n_q + 2 * p.n_kv) * D + (size_t)Jp * p.n_q * D + (size_t)hp * step_lse_words(Jp) + 2 * jp;
    const uint32_t ninf = c.tagw | 0xFC00u;
    st_tagged(Eo + tid, c.tagw | (uint32_t)__half_as_ushort(__float2half(o / L)));
    if (tid == 0) {   // log-sum-exp of the slice as an fp16 value and the fp16 remainder
      const float lse = M + __logf(L);
      const half hi = __float2half(lse), lo = __float2half(lse - __half2float(hi));
      st_tagged(El, c.tagw | (uint32_t)__half_as_ushort(hi));
      st_tagged(El + 1, c.tagw | (uint32_t)__half_as_ushort(lo));
      if ((Jp & 1) && jp == Jp - 1) { st_tagged(El + 2, ninf); st_tagged(El + 3, c.tagw); }
    }
  }
  stamp(c, trace_at + 2);
  consumer_sync();
}

}  // namespace

// ---- the kernel ------------------------------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const __grid_constant__ StepParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  Cta c;
  c.smem = smem;
  c.p = &p;
  // the per-layer pointer table, copied once from global memory: every phase starts from these pointers, and a
  // global load in front of each would put an L2 round trip on the critical path ~10 times per layer
  StepLayer* lys = reinterpret_cast<StepLayer*>(smem + p.off_table);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int cta = blockIdx.x, ncta = gridDim.x;

  if (tid == 0) {
    for (int i = 0; i < p.ns; ++i) { mbar_init(c.full(i), 1); mbar_init(c.empty(i), kNCW); }
    *c.abort() = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const int n_qkv = (p.n_q + 2 * p.n_kv) * p.D, n_att = p.n_q * p.D;
  // This CTA's tiles of the five matrix shapes of a step (qkv, o, gate|up, down, head): computed once (they involve
  // integer divisions) and kept in shared memory for producer and consumers.
  Slice* sl = reinterpret_cast<Slice*>(smem + 512);
  if (tid < 5) {
    const int rows = tid == 0 ? n_qkv : (tid == 2 ? p.I : (tid == 4 ? p.V : p.H));
    sl[tid] = slice_of(rows, tid == 2, cta, ncta);
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
  // Context slices per query head in attention (the exchange layout always has room for J). Slicing pays from about
  // 1200 cached tokens on: below that the K/V copies of 96 more CTAs delay the weight stream (an SM's copy engine takes
  // ~1 us for the 16 page copies of a stage) and the merge costs the o projection's staging a second trip through
  // the L2, which together outweigh a fold that is shorter by one or two stages. In a step below the threshold slice
  // 0 takes the whole context and the others publish empty partials (every exchange word is rewritten in every
  // step - the tag invariant - but nobody waits for these). Every CTA reads the same pos, so all agree.
  const int J = p.att_slices;
  const bool sliced = pos >= kSliceMinContext && J > 1;
  const int per_layer = (int)step_words_per_layer(p.H, p.I, p.n_q, p.n_kv, p.D, J);   // exchange words per layer

  if (warp == kNCW) {
    // ================= producer =================
    RingPos rp = {0, 1u, 0};   // parity 1: the first pass over a fresh `empty` barrier does not wait
    for (int l = 0; l < p.L && !*c.abort(); ++l) {
      const StepLayer& ly = lys[l];
      const Mat mats[4] = {{(const uint8_t*)ly.w[0], n_qkv, p.H, 0},
                           {(const uint8_t*)ly.w[1], p.H, n_att, 0},
                           {(const uint8_t*)ly.w[2], p.I, p.H, 1},
                           {(const uint8_t*)ly.w[3], p.H, p.I, 0}};
      produce(c, mats[0], sl[0], rp, lane);
      for (int u = cta; u < p.n_q * J && !*c.abort(); u += ncta)   // attention unit u: head u % n_q, slice u / n_q
        if (sliced || u < p.n_q) produce_kv(c, p, ly, (u % p.n_q) / hpg, u / p.n_q, sliced ? J : 1, pos, rp, lane);
#pragma unroll
      for (int k = 1; k < 4; ++k)
        if (!*c.abort()) produce(c, mats[k], sl[k], rp, lane);
    }
    if (!*c.abort()) {
      const Mat head = {(const uint8_t*)p.w_head, p.V, p.H, 0};
      produce(c, head, sl[4], rp, lane);
    }
    // Leave only when every copy issued has landed. On the normal path the consumers have waited on every full
    // barrier already; on abort, wait (bounded) for the full barriers of the stages still in the ring.
    if (*c.abort()) {
      const int it = rp.count;
      for (int k = max(0, it - c.p->ns); k < it; ++k) {
        const int slot = k % c.p->ns;
        for (int i = 0; i < kSpinLimit; ++i)
          if (mbar_try_wait(c.full(slot), (k / c.p->ns) & 1)) break;
      }
    }
    return;
  }

  // ================= consumers =================
#ifdef B200_STEP_TRACE
  // trace row of a CTA: kTraceHead slots (0 = start, 1 = keys exchanged, 2 = token written), then per layer
  // kTracePerLayer: per phase {staged, first weights there, GEMV done, barrier passed, emitted}, then attention
  // {q k v polled and rotated, cached tokens folded, warps merged and output stored, done, wait for K/V stages};
  // the LM head uses the slots of a layer L
  c.tr = p.trace ? p.trace + (size_t)cta * (kTraceHead + kTracePerLayer * (p.L + 1)) : nullptr;
#endif
  stamp(c, 0);
  RingPos rp = {0, 0u, 0};
  unsigned long long best = 0ull;
  // RoPE factors and the page of this step's token depend only on pos: the attention CTAs fetch them now, off the
  // critical path, into the attention scratch (first read two barriers into the first attention phase)
  if (cta < p.n_q * J) {
    float* rope = c.att() + 4 * p.D + kNCW * p.D + 2 * kNCW;
    if (tid < (p.D >> 1)) {
      rope[tid] = p.cos_t[(size_t)pos * (p.D >> 1) + tid];
      rope[(p.D >> 1) + tid] = p.sin_t[(size_t)pos * (p.D >> 1) + tid];
    }
    if (tid == 0) reinterpret_cast<int*>(rope)[p.D] = p.bt[pos >> p.log2P];
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
    uint32_t *Eqkv = E, *Eatt = E + n_qkv, *Else = Eatt + (size_t)J * n_att;
    uint32_t *Eo = Else + p.n_q * step_lse_words(J), *Eact = Eo + p.H, *Edown = Eact + p.I;
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
    const Slice s = sl[is_head ? 4 : ph];
    // the layers alternate between two partial-sum buffers (a slow thread may still add up phase n while a fast warp
    // writes phase n + 1); the head, last and largest, takes the whole area
    const int pstride = is_head ? p.part_stride_head : p.part_stride;
    float* part = c.part() + ((step & 1) && !is_head ? kNCW * p.part_stride : 0);
    if (nw) {
      const half* emb_row = nullptr;
      if (step == 0) {
        // A token id outside the embedding table (a caller's mistake) must not become an address: row 0 is read
        // instead and the step reports it.
        long long tok_in = p.tok[0];
        if (tok_in < 0 || tok_in >= p.V) {
          if (cta == 0 && tid == 0) atomicCAS(&p.ctrl->error, 0, ERR_TOKEN);
          tok_in = 0;
        }
        emb_row = p.emb + (size_t)tok_in * p.H;
      }
      stage_norm(c, Ein, emb_row, nw, n_in, p.eps, warp, lane);
    }
    else if (s.nt > 0) {
      if (ph == 1 && sliced) stage_attn(c, Eatt, Else, J, n_att, p.D, warp, lane);
      else stage_plain(c, Ein, n_in, warp, lane);   // one slice: its normalised output is the attention output
    }
    const int tr_at = kTraceHead + kTracePerLayer * l + kTracePerPhase * ph;
    stamp(c, tr_at);
    gemv(c, m, s, part, pstride, rp, warp, lane, tr_at + 1);
    stamp(c, tr_at + 2);
    if (consumer_sync_or(*c.abort())) return;
    stamp(c, tr_at + 3);
    reduce_emit(c, m, s, part, pstride, out, Eout, p.logits, best, tid);
    stamp(c, tr_at + 4);
    if (is_head) break;
    if (ph == 0) {
      for (int u = cta; u < p.n_q * J; u += ncta) {
        attention_head<D>(c, p, ly, E, u, pos, rp, tid, kTraceHead + kTracePerLayer * l + 4 * kTracePerPhase);
        if (consumer_sync_or(*c.abort())) return;
      }
      stamp(c, kTraceHead + kTracePerLayer * l + 4 * kTracePerPhase + 3);
    }
  }
  // this CTA's candidate: max over its threads' keys
  unsigned long long* keys = reinterpret_cast<unsigned long long*>(c.att());
  {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
      best = other > best ? other : best;
    }
  }
  if (lane == 0) keys[warp] = best;
  if (consumer_sync_or(*c.abort())) return;
  stamp(c, 1);
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
    if (tid == 0 && !*c.abort()) {
      for (int k = 0; k < kNCW; ++k) b = keys[kNCW + k] > b ? keys[kNCW + k] : b;
      // b == 0: no logit was comparable (all NaN). torch.argmax, which the reference uses, answers with a valid
      // index in that case; token 0 is this kernel's answer.
      const long long t = b ? (long long)(0x7FFFFFFF - (int)(b & 0xFFFFFFFFu)) : 0ll;
      p.tok[0] = t;
      if (p.history) p.history[pos] = t;
      p.pos[0] = pos + 1;
      p.ctrl->epoch = epoch;
      stamp(c, 2);
    }
  }
}

// Lays the fixed areas out behind the header (sizes in, offsets out); returns where the ring starts.
size_t decode_step_plan_smem(StepParams& p, int resid_bytes, int xin_bytes, int xsum_bytes, int att_bytes,
                             int part_bytes, int table_bytes) {
  p.off_xin = kHeaderBytes + resid_bytes;
  p.off_xsum = p.off_xin + xin_bytes;
  p.off_att = p.off_xsum + xsum_bytes;
  p.off_part = p.off_att + att_bytes;
  p.off_table = p.off_part + part_bytes;
  p.off_ring = p.off_table + table_bytes;
  return (size_t)p.off_ring;
}
int decode_step_threads() { return kThreads; }
int decode_step_max_stages() { return kMaxStages; }
int decode_step_consumer_warps() { return kNCW; }
int decode_step_max_kv_tokens() { return kMaxKvTokens; }

cudaError_t decode_step_launch(const StepParams& p, int grid, size_t smem, cudaStream_t st) {
  // the shared-memory limit of a kernel is a per-device attribute
  static bool configured[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    e = cudaFuncSetAttribute(decode_step_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(decode_step_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 64) configured[dev] = true;
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

}  // namespace b200
