#pragma once
// Tensor-core variant of the fused TimestepNorm -> causal EMA (and of the EMA alone, and of
// TimestepNorm alone) for bf16 activations with contiguous channels, with or without a padding mask.
//
// Work split.  A CTA owns kCg column groups (8 channels = 16 bytes each; kCg = 8, 7, 4 or 2) of 8
// sequences and walks time in steps of 32 positions.  Warp w owns column group w (or, with two
// warps per column group, four of its eight channels).  For one
// channel the 8 sequences x 2 consecutive 16-position chunks of a step form the 16 rows of
// warp-level MMAs (row g = sequence g, chunk 0; row g + 8 = sequence g, chunk 1), so every carry
// between chunks stays inside one thread and no cross-lane scan is needed.  The 56-channel tile
// exists for load balance: one CTA fits per SM, and e.g. 2048 channels x 64 sequences give
// 37 x 8 = 296 CTAs = exactly two waves over 148 SMs (64-channel tiles leave 40 SMs idle in the
// second wave).
//
// Math per channel and step (h = pole states, C = 16):
//   TimestepNorm : with c the running mean at the start of the step and d = x - c, the prefix
//                  sums of x and d^2 inside each half chunk are products with a 0/1 triangular
//                  matrix (one tf32 MMA per half); the totals of the halves are the last prefixes,
//                  handed round by a shuffle, and the running totals are added in fp32.  Centring
//                  keeps mean^2 small against the variance, so the tf32 truncation of the MMA
//                  inputs (11 significant bits) only costs ~2^-11 of the variance.  Then
//                  u = sum(x)/n - c, var = (M2 + sum(d^2))/n - u^2, xn = (d - u) * rstd * w + b.
//                  MMAs that depend on one another are what a warp waits for (two warps per
//                  scheduler cannot hide it), so no MMA here consumes another MMA's result.
//   EMA          : y = T xn + G h_start   (T: 16x16 lower-triangular Toeplitz of the kernel
//                  k[l] = sum_n p g q^l, omega folded into k[0]; G[t][n] = g q^(t+1))
//                  h_local = P xn          (P[n][t] = p q^(15-t));  h_next = q^16 h + h_local.
// The per-channel matrices T, P, G are built once per CTA, in MMA fragment order, in shared
// memory.  Tiles move by TMA (128-byte swizzle), are transformed in place and stored by TMA.
//
// Forms of the kernel (template parameters): with or without the normalisation; with or without
// the EMA (TimestepNorm alone); SiLU epilogue; one or two warps per 16-byte column; a second
// output with the normalised activations (what the Mega block feeds its value projection);
// complex poles (MultiHeadComplexEMA: P yields Re and Im of the local states, the carry is a
// complex multiply by q^16, G takes Re(gamma q^(t+1)) against Re h and -Im(...) against Im h);
// a padding mask; groups of warps pipelined along the sequence (problems with few strips); the
// sequence cut into runs that separate CTAs take one after the other (problems of more than one
// wave of CTAs).  Each is described at the kernel.
#include <mutex>
#include <string>
#include <type_traits>
#include <utility>

#include "common.cuh"
#include "stream_cl.cuh"
#include "tma.cuh"

namespace mega {

namespace {

constexpr int kSeq = 8;    // sequences per CTA
constexpr int kStep = 32;  // positions per step (2 chunks of 16)

// kXn: the kernel also writes the normalised activations (the Mega block feeds them to its value
// projection): two more tile buffers, filled from registers and stored by TMA like the outputs, at
// the price of one stage of the ring.
// kCplx: complex poles (MultiHeadComplexEMA): P, G and q^16 hold real and imaginary parts.
// kWp: pipeline depth along the sequence (see the kernel): kWp groups of warps work on kWp
// consecutive steps of the same strip at once and hand the running quantities over through
// per-warp mailboxes in shared memory.
// kSm: (kWp == 1) the running quantities of a warp live in its shared-memory mailbox between steps
// instead of in registers (56 registers of a thread that only hold state).
template <int kCg, bool kXn = false, bool kCplx = false, int kWs = 1, int kWp = 1, bool kSm = false>
struct Cfg {
  static constexpr bool kMail = kWp > 1 || kSm;
  static constexpr int kCm = kCplx ? 2 : 1;
  // Ring depth: a tile is fetched kStages - kWp steps before it is used.  Without the pipeline
  // deeper rings were measured and do not pay: a fifth stage leaves the SM too little L1 for the
  // few spilled registers.  With it a tile is small (narrow tiles only) and the ring holds three
  // rounds of the pipeline.
  static constexpr int kStages = kWp > 1 ? 3 * kWp : ((kXn || kSm) ? 3 : 4);
  static constexpr int kWarps = kCg * kWs * kWp;
  static constexpr int kE = 8 / kWs;  // channels per warp
  static constexpr int kCh = kCg * 8;                       // channels per CTA
  static constexpr int kRow = kCg * 16;                     // bytes per tile row
  static constexpr int kStageBytes = kSeq * kStep * kRow;   // 32 KiB (kCg = 8) / 28 KiB (kCg = 7)
  static constexpr int kOffStages = 0;
  static constexpr int kOffXn = kOffStages + kStages * kStageBytes;  // kXn: [2][stage] normalised tiles
  static constexpr int kOffT = kOffXn + (kXn ? 2 * kStageBytes : 0);  // [kCh][2][32] u32
  static constexpr int kOffP = kOffT + kCh * 2 * 32 * 4;            // [kCh][kCm][32] uint4
  static constexpr int kOffG = kOffP + kCm * kCh * 4 * 32 * 4;      // [kCh][kCm][32] uint4
  static constexpr int kOffA = kOffG + kCm * kCh * 4 * 32 * 4;      // [kCh][16] f32 (q^16; kCplx: float2)
  static constexpr int kOffWB = kOffA + kCm * kCh * 16 * 4;         // [kCh] {w, w, b, b} f32 (pairs as the packed operations take them)
  static constexpr int kOffKp = kOffWB + kCh * 4 * 4;               // [kCh][16] f32 scratch: kernel taps
  static constexpr int kOffBar = kOffKp + kCh * 16 * 4;             // full[kStages], done[kStages], xfree[2], abort word
  // mailboxes (kWp > 1): per warp, per kind (0: statistics, 1: pole states), per channel: 32 lanes x
  // 16 bytes of data, and one mbarrier whose phases count the steps that have been posted
  static constexpr int kOffMail = (kOffBar + (2 * kStages + 2) * 8 + 16 + 15) / 16 * 16;
  static constexpr int kMailWarp = 2 * kE * 32 * 16;
  static constexpr int kOffFlag = kOffMail + (kMail ? kWarps * kMailWarp : 0);
  static constexpr int kFlagWarp = 2 * kE * 8;  // one mbarrier per kind and channel: "this step's value is posted"
  static constexpr int kSmemBytes = kOffFlag + (kWp > 1 ? kWarps * kFlagWarp : 0) + 1024;  // + alignment slack
  static_assert(kSmemBytes <= 227 * 1024, "tile does not fit the shared memory of an SM");
};

// d = a * b + c (c read-only, so a zero or shared accumulator input needs no copy)
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1, float c0, float c1, float c2, float c3) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c0), "f"(c1), "f"(c2), "f"(c3));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], float a0, float a1, float a2, float a3, float b0,
                                         float b1, float c0, float c1, float c2, float c3) {
  asm(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(__float_as_uint(a0)), "r"(__float_as_uint(a1)), "r"(__float_as_uint(a2)),
        "r"(__float_as_uint(a3)), "r"(__float_as_uint(b0)), "r"(__float_as_uint(b1)), "f"(c0), "f"(c1),
        "f"(c2), "f"(c3));
}
// shared-memory accesses by 32-bit shared address (keeps them LDS/STS rather than generic).  `off`
// must be a compile-time constant after inlining: it becomes the immediate of the instruction, so
// that a thread keeps one base register per array instead of computing every address.
template <int kOff = 0>
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(kOff));
  return v;
}
template <int kOff = 0>
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(kOff));
  return v;
}
template <int kOff = 0>
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(kOff));
  return v;
}
template <int kOff = 0>
__device__ __forceinline__ void sts64(uint32_t addr, uint2 v) {
  asm volatile("st.shared.v2.u32 [%0+%1], {%2,%3};" ::"r"(addr), "n"(kOff), "r"(v.x), "r"(v.y) : "memory");
}
template <int kOff = 0>
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0+%1], {%2,%3,%4,%5};" ::"r"(addr), "n"(kOff), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Compile-time loop: f(std::integral_constant<int, 0>{}), ..., so that the body can use its index
// in constant expressions (instruction immediates).
template <int... Is, typename F>
__device__ __forceinline__ void static_for_impl(std::integer_sequence<int, Is...>, F&& f) {
  (f(std::integral_constant<int, Is>{}), ...);
}
template <int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  static_for_impl(std::make_integer_sequence<int, N>{}, f);
}
// The abort word in shared memory, and the hand-off between the warps of a pipeline.  A warp posts a
// value for its successor by writing the data to its mailbox and arriving (every lane, release
// semantics) on the mailbox's mbarrier; the successor waits for the phase of that step and reads
// the data (each lane only reads what the same lane of the other warp wrote).  A waiting warp is
// suspended by the hardware inside mbarrier.try_wait instead of spinning on a flag.
__device__ __forceinline__ uint32_t ld_volatile_s(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.volatile.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_s(uint32_t addr, uint32_t v) {
  asm volatile("st.volatile.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
template <int kOff = 0>
__device__ __forceinline__ void mbar_arrive_s(uint32_t addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0+%1];" ::"r"(addr), "n"(kOff) : "memory");
}
template <int kOff = 0>
__device__ __forceinline__ bool mbar_try_s(uint32_t addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1+%2], %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(addr), "n"(kOff), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait for a phase of an mbarrier (out of line: the caller tries once inline and comes here
// only when it has to wait).  Gives up when the CTA's abort word is set (another waiter has given
// up) or after `limit` SM cycles; then it raises the device error word, sets the abort word and
// returns false.
__device__ __noinline__ bool mbar_wait_slow(uint32_t addr, uint32_t parity, uint32_t abort_addr, long long limit) {
  const long long start = clock64();
  while (true) {
    if (mbar_try_s(addr, parity)) return true;
    if (ld_volatile_s(abort_addr) != 0) return false;
    if (clock64() - start > limit) {
      g_device_error = 2;
      st_volatile_s(abort_addr, 1u);
      return false;
    }
  }
}
// mbar_wait with the caller's cycle limit and the CTA's abort word (same give-up rule as poll_flag).
__device__ __forceinline__ bool mbar_wait_lim(uint64_t* bar, uint32_t parity, uint32_t abort_addr, long long limit) {
  const uint32_t addr = smem_u32(bar);
  uint32_t ok = 0;
  long long start = 0;
  for (int spins = 0;; ++spins) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if (spins == 0) start = clock64();
    if (ld_volatile_s(abort_addr) != 0) return false;
    if (clock64() - start > limit) {
      g_device_error = 1;
      st_volatile_s(abort_addr, 1u);
      return false;
    }
  }
}
// two fp32 -> packed bf16x2 (lo in the low half)
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float rsqrt_fast(float v) {
  float r;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float rcp_fast(float v) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
  return r;
}
__device__ __forceinline__ float qpow(float logq, bool qpos, int l) {
  return l == 0 ? 1.0f : (qpos ? __expf((float)l * logq) : 0.0f);
}
// (qr + i qi)^l
__device__ __forceinline__ float2 cpow(float qr, float qi, int l) {
  if (l == 0) return make_float2(1.f, 0.f);
  const float rho = hypotf(qr, qi);
  if (!(rho > 0.f)) return make_float2(0.f, 0.f);
  const float mag = __expf((float)l * __logf(rho));
  float sn, cs;
  sincosf((float)l * atan2f(qi, qr), &sn, &cs);
  return make_float2(mag * cs, mag * sn);
}
__device__ __forceinline__ uint32_t bf16_bits(float v) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Byte offset of the 16-byte vector (sequence, position, column group) inside a stage.  kCg = 8:
// rows are 128 bytes and TMA applies its 128-byte swizzle (chunk index XOR row mod 8); kCg = 7:
// rows are 112 bytes, unswizzled (the odd pitch already staggers the banks); kCg = 4, 2 (the
// narrow tiles of small problems): 64- and 32-byte rows, unswizzled.
template <int kCg>
__device__ __forceinline__ uint32_t vec_off(int seq, int t, int cg) {
  const int row = seq * kStep + t;
  if (kCg == 8) return (uint32_t)(row * 128 + ((cg ^ (row & 7)) << 4));
  return (uint32_t)(row * (kCg * 16) + (cg << 4));
}

// kWs = warps per column group: 1 (a warp owns the 8 channels of its 16-byte column) or 2 (a warp
// owns 4 of them: half the per-thread state and tile registers, so more warps fit an SM).
// kEma = false: TimestepNorm alone (y = the normalised activations; no pole matrices, no states).
// kWp = pipeline depth along the sequence.  A strip (8 sequences x the channels of a warp) is a
// serial chain over the steps, so a problem with few strips leaves the SMs short of warps.  With
// kWp > 1 the CTA holds kWp groups of warps; group w takes the steps i = w, w + kWp, ... of every
// strip and the running quantities (sum and squared deviations of TimestepNorm, pole states) travel
// from the warp of step i to the warp of step i + 1 through a mailbox in shared memory, per channel
// and as soon as they are known: the statistics right after the prefix sums of a channel (the sums
// of squares are taken about a centre the warp already holds, its own latest mean, and moved to the
// incoming mean afterwards), the pole states right after the local-state product.  The warps of
// consecutive steps thus run a few hundred cycles apart instead of a whole step.
// kMask: a padding mask (B, L) is honoured as TimestepNorm defines it: a padded position does not
// advance the statistics and its normalised value is 0 (so it feeds 0 to the EMA, whose state just
// decays across it); positions past the end of a ragged last step count as padded.  Per step a warp
// turns the mask bytes of its 8 sequences x 32 positions into 0/1 flags, takes their prefix counts
// with the same triangular MMA as the sums (the divisor of the running mean at each position), and
// multiplies the inputs of the sums and the normalised values by the flags.
// kPs: segmented form for problems of more than one wave of CTAs.  A strip is a serial chain along
// the sequence, so a grid of (tile, group of sequences) CTAs runs in whole waves: 256 CTAs of 8 warps
// on 148 SMs take two waves although they are 1.73 waves of work.  Here the sequence is cut into
// n_seg runs and the grid has one CTA per work item (run, tile, group).  A CTA draws its item from a
// counter when it starts, so the items are taken in run-major order by CTAs that are running, and
// an item starts from the statistics and pole states that the item of the run before left in
// global memory (the call's own mean / variance outputs, and h_out or a hand-off buffer) once that
// item's flag is set.  An item depends on one that was drawn earlier, by a CTA that is running or
// done, so the waits end; they are bounded like every other wait of this kernel.  The SMs stay
// busy because the hardware hands the next CTA to whichever SM becomes free.  A CTA lives for one
// run only, so its set-up counts: the matrices of each tile of channels are built once, by a launch
// of this kernel in its builder form (kPs == 2: set-up only, the shared-memory image of the
// matrices copied to global memory), and the CTAs of the runs (kPs == 1) fetch that image with a
// bulk copy instead of building it.  (kPs == 3: the CTAs of the runs build their matrices themselves;
// kept for the normalising form, whose step loop the compiler allocates better that way.)
template <bool kNorm, int kCg, bool kSilu, int kWs, bool kXn, bool kEma = true, bool kCplx = false, int kWp = 1,
          bool kMask = false, bool kSm = false, int kPs = 0>
__global__ void __launch_bounds__(kCg * kWs * kWp * 32, 1)
    tsn_ema_mma_kernel(const __grid_constant__ CUtensorMap tmx, const __grid_constant__ CUtensorMap tmy,
                       const __grid_constant__ CUtensorMap tmn, StreamArgs a) {
  static_assert(!kXn || kNorm, "the normalised copy exists only with the normalisation");
  static_assert(kEma || (kNorm && !kXn && !kSilu), "without the EMA the kernel is the plain normalisation");
  static_assert(!kCplx || kEma, "complex poles need the EMA");
  static_assert(kWp == 1 || (!kXn && !kCplx && kEma), "the pipelined form covers the real EMA without the second output");
  static_assert(!kMask || (kWp == 1 && !kCplx && !(kXn && !kNorm)), "masks: real poles, not pipelined");
  static_assert(!kSm || (kWp == 1 && !kXn && !kCplx && kEma && !kMask), "state in shared memory: the plain real form");
  static_assert(!kPs || (kWp == 1 && kWs == 1 && !kXn && !kCplx && !kMask && !kSm), "segmented: the plain real form");
  static_assert(kPs == 0 || kPs == 3 || kEma, "pre-built matrices exist for the EMA only");

  using C = Cfg<kCg, kXn, kCplx, kWs, kWp, kSm>;
  constexpr bool kMail = C::kMail;   // running quantities travel through / live in the mailboxes
  constexpr bool kLate = kWp > 1;    // ... and arrive from another warp, after this warp's own sums
  constexpr int kCh = C::kCh;
  constexpr int kCm = C::kCm;
  constexpr int kThreads = kCg * kWs * kWp * 32;
  constexpr int kGroup = kCg * kWs;  // warps of one pipeline group
  constexpr int kStages = C::kStages;
  constexpr int kE = 8 / kWs;   // channels per warp
  constexpr int kVw = kE / 2;   // 32-bit words (channel pairs) per tile vector of this warp
  constexpr int kStageBytes = C::kStageBytes;
  constexpr int kOffStages = C::kOffStages, kOffT = C::kOffT, kOffP = C::kOffP, kOffG = C::kOffG;
  constexpr int kOffA = C::kOffA, kOffWB = C::kOffWB, kOffKp = C::kOffKp, kOffBar = C::kOffBar;
  constexpr int kMatBytes = C::kOffKp - C::kOffT;   // T, P, G, q^16 and the affine pair of a tile
  static_assert(kMatBytes % 16 == 0 && C::kOffT % 16 == 0, "bulk copies move 16-byte units");
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint32_t* Tc = reinterpret_cast<uint32_t*>(sm + kOffT);
  uint4* Pc = reinterpret_cast<uint4*>(sm + kOffP);
  uint4* Gc = reinterpret_cast<uint4*>(sm + kOffG);
  float* Ac = reinterpret_cast<float*>(sm + kOffA);
  float* WB = reinterpret_cast<float*>(sm + kOffWB);
  float* Kp = reinterpret_cast<float*>(sm + kOffKp);
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint64_t* done = full + kStages;  // one arrival per warp once its slice of the stage is written
  uint64_t* xfree = done + kStages;  // kXn: buffer k of the normalised tiles has been read by its store

  const uint32_t sm_s = smem_u32(sm);
  const uint32_t abort_s = sm_s + kOffBar + (2 * kStages + 2) * 8;  // set when a bounded wait gave up
  // kPs: the work item of this pass, its last step + 1 and (ring position - step), kept here rather
  // than in registers that would be live across the whole step loop
  const uint32_t item_s = abort_s + 4, iend_s = abort_s + 8, delta_s = abort_s + 12;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wp = (tid >> 5) / kGroup;            // pipeline group: takes the steps i = wp (mod kWp)
  const int wig = (tid >> 5) % kGroup;           // warp inside its group
  const int warp = wig / kWs;  // column group
  const int hf = wig % kWs;    // which part of the column's channels
  const bool issuer = tid == wp * kGroup * 32;  // moves the tiles of this group's steps
  const long long wait_limit = a.wait_limit;
  // mailboxes: this warp writes its own, and reads that of the same strip's warp one group before
  const uint32_t mail_out = sm_s + C::kOffMail + (uint32_t)(tid >> 5) * C::kMailWarp + lane * 16;
  const uint32_t flag_out = sm_s + C::kOffFlag + (uint32_t)(tid >> 5) * C::kFlagWarp;
  const int wprev = kSm ? (tid >> 5) : ((wp + kWp - 1) % kWp) * kGroup + wig;
  const uint32_t mail_in = sm_s + C::kOffMail + (uint32_t)wprev * C::kMailWarp + lane * 16;
  const uint32_t flag_in = sm_s + C::kOffFlag + (uint32_t)wprev * C::kFlagWarp;
  const int g = lane >> 2, q = lane & 3;
  int d0 = blockIdx.x * kCh;   // (kPs: set per work item)
  int b0 = blockIdx.y * kSeq;
  const int L = a.L;
  const int nsteps = (L + kStep - 1) / kStep;
  int i_begin = 0, i_end = nsteps;  // steps of this CTA (kPs: those of its run)
  int seg = 0;

  if (tid == 0) {
    prefetch_tensormap(&tmx);
    prefetch_tensormap(&tmy);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], kCg * kWs);
    }
    if (kXn) {
      mbar_init(&xfree[0], 1);
      mbar_init(&xfree[1], 1);
    }
    if (kPs == 1) mbar_init(&xfree[0], 1);   // (here: the bulk copy of the matrices)
    st_volatile_s(abort_s, 0u);
    if (kWp > 1) {  // hand-off barriers: all 32 lanes of the posting warp arrive
      for (int k = 0; k < C::kWarps * 2 * C::kE; ++k)
        mbar_init(reinterpret_cast<uint64_t*>(sm + C::kOffFlag) + k, 32);
    }
    mbar_fence_init();
  }
  if constexpr (kPs == 1 || kPs == 3) {
    if (tid == 0) st_volatile_s(item_s, (uint32_t)atomicAdd(a.sched, 1));
  }
  __syncthreads();
  if constexpr (kPs == 1 || kPs == 3) {
    const int item = (int)ld_volatile_s(item_s);   // (< n_items: the grid has one CTA per item)
    const int n_grp = a.n_items / a.n_seg;
    seg = item / n_grp;
    const int grp = item - seg * n_grp;
    d0 = (grp % a.tiles_d) * kCh;
    b0 = (grp / a.tiles_d) * kSeq;
    i_begin = seg * a.seg_steps;
    i_end = min(nsteps, i_begin + a.seg_steps);
    if (tid == 0) {
      st_volatile_s(iend_s, (uint32_t)i_end);
      st_volatile_s(delta_s, (uint32_t)(0 - i_begin));
    }
    // (visible to all after the barrier between the two phases of the matrices below)
  }
  if (tid == 0 && kPs != 2) {
    if constexpr (kPs == 1) {
      const unsigned char* src = a.matrices + (size_t)(d0 / kCh) * kMatBytes;
      mbar_expect_tx(&xfree[0], kMatBytes);
      for (int o = 0; o < kMatBytes; o += 32768)
        bulk_load_1d(sm + kOffT + o, src + o, (uint32_t)min(32768, kMatBytes - o), &xfree[0]);
    }
    for (int s = 0; s < kStages - kWp && i_begin + s < i_end; ++s) {
      const int s2 = s;
      mbar_expect_tx(&full[s2], kStageBytes);
      if (i_begin + s != a.withhold_step)
        tma_load_3d(sm + kOffStages + s2 * kStageBytes, &tmx, d0, (i_begin + s) * kStep, b0, &full[s2]);
    }
  }

  // ---- per-channel matrices, phase 1: kernel taps k'[l], q^16, affine ---------------------
  for (int it = tid; kPs != 1 && it < kCh * 16; it += kThreads) {
    const int ch = it >> 4, l = it & 15;
    const int d = d0 + ch;
    float acc = 0.f, a16 = 0.f, a16i = 0.f;
    if (kEma && d < a.D) {
      for (int n = 0; n < a.N; ++n) {
        const size_t c = (size_t)d * a.N + n;
        const float pn = __ldg(a.p + c);
        if (kCplx) {  // k[l] = sum_n p Re(gamma q^l)
          const float qr = __ldg(a.q + 2 * c), qi = __ldg(a.q + 2 * c + 1);
          const float2 ql = cpow(qr, qi, l);
          acc = fmaf(pn, __ldg(a.g + 2 * c) * ql.x - __ldg(a.g + 2 * c + 1) * ql.y, acc);
          if (n == l) {
            const float2 q16 = cpow(qr, qi, 16);
            a16 = q16.x;
            a16i = q16.y;
          }
        } else {
          const float qn = __ldg(a.q + c), gn = __ldg(a.g + c);
          const bool qpos = qn > 0.f;
          const float lq = qpos ? __logf(qn) : 0.f;
          acc = fmaf(pn * gn, qpow(lq, qpos, l), acc);
          if (n == l) a16 = qpow(lq, qpos, 16);
        }
      }
      if (l == 0) acc += __ldg(a.omega + d);
    }
    Kp[it] = acc;
    if (kCplx) {
      Ac[2 * it] = a16;
      Ac[2 * it + 1] = a16i;
    } else {
      Ac[it] = a16;  // entry (ch, pole l); poles >= a.N stay 0
    }
    if (l < 2) {
      float v = (l == 0) ? 1.f : 0.f;
      if (kNorm && d < a.D) v = (l == 0) ? __ldg(a.gamma + d) : __ldg(a.beta + d);
      if (!kNorm && kMask && kEma && l == 0 && d < a.D) v = __ldg(a.omega + d);   // see the masked EMA epilogue
      WB[ch * 4 + 2 * l] = v;
      WB[ch * 4 + 2 * l + 1] = v;
    }
  }
  __syncthreads();
  // ---- phase 2: fragment-ordered T, P, G --------------------------------------------------
  for (int it = tid; kEma && kPs != 1 && it < kCh * 32; it += kThreads) {
    const int ch = it >> 5, ln = it & 31;
    const int gg = ln >> 2, qq = ln & 3;
    const int d = d0 + ch;
    // Toeplitz: B[k = t][n = t'] = k'[t' - t]; R0: t' = gg, t = 2qq, 2qq+1; R1: t' = 8 + gg
    auto tap = [&](int l) -> float { return (l >= 0 && l < 16) ? Kp[ch * 16 + l] : 0.f; };
    Tc[(ch * 2 + 0) * 32 + ln] = bf16_bits(tap(gg - 2 * qq)) | (bf16_bits(tap(gg - 2 * qq - 1)) << 16);
    Tc[(ch * 2 + 1) * 32 + ln] = bf16_bits(tap(8 + gg - 2 * qq)) | (bf16_bits(tap(8 + gg - 2 * qq - 1)) << 16);
    if (kCplx) {
      // the same fragments with complex powers: P gives Re and Im of the local states, G takes
      // Re(gamma q^(t'+1)) against Re h and -Im(gamma q^(t'+1)) against Im h
      uint32_t prr[4], pri[4], grr[4], gri[4];
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const int n = 8 * nb + gg;
        float pn = 0.f, qr = 0.f, qi = 0.f;
        if (d < a.D && n < a.N) {
          const size_t c = (size_t)d * a.N + n;
          pn = __ldg(a.p + c);
          qr = __ldg(a.q + 2 * c);
          qi = __ldg(a.q + 2 * c + 1);
        }
        const float2 e0 = cpow(qr, qi, 15 - 2 * qq), e1 = cpow(qr, qi, 14 - 2 * qq);
        const float2 e2 = cpow(qr, qi, 7 - 2 * qq), e3 = cpow(qr, qi, 6 - 2 * qq);
        prr[nb * 2 + 0] = bf16_bits(pn * e0.x) | (bf16_bits(pn * e1.x) << 16);
        pri[nb * 2 + 0] = bf16_bits(pn * e0.y) | (bf16_bits(pn * e1.y) << 16);
        prr[nb * 2 + 1] = bf16_bits(pn * e2.x) | (bf16_bits(pn * e3.x) << 16);
        pri[nb * 2 + 1] = bf16_bits(pn * e2.y) | (bf16_bits(pn * e3.y) << 16);
        const int tp = 8 * nb + gg;
        float cr[4], ci[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int pole = 2 * qq + (k & 1) + ((k >> 1) << 3);
          cr[k] = ci[k] = 0.f;
          if (d < a.D && pole < a.N) {
            const size_t c = (size_t)d * a.N + pole;
            const float2 w = cpow(__ldg(a.q + 2 * c), __ldg(a.q + 2 * c + 1), tp + 1);
            const float gre = __ldg(a.g + 2 * c), gim = __ldg(a.g + 2 * c + 1);
            cr[k] = gre * w.x - gim * w.y;
            ci[k] = -(gre * w.y + gim * w.x);
          }
        }
        grr[nb * 2 + 0] = bf16_bits(cr[0]) | (bf16_bits(cr[1]) << 16);
        grr[nb * 2 + 1] = bf16_bits(cr[2]) | (bf16_bits(cr[3]) << 16);
        gri[nb * 2 + 0] = bf16_bits(ci[0]) | (bf16_bits(ci[1]) << 16);
        gri[nb * 2 + 1] = bf16_bits(ci[2]) | (bf16_bits(ci[3]) << 16);
      }
      Pc[(ch * 2 + 0) * 32 + ln] = make_uint4(prr[0], prr[1], prr[2], prr[3]);
      Pc[(ch * 2 + 1) * 32 + ln] = make_uint4(pri[0], pri[1], pri[2], pri[3]);
      Gc[(ch * 2 + 0) * 32 + ln] = make_uint4(grr[0], grr[1], grr[2], grr[3]);
      Gc[(ch * 2 + 1) * 32 + ln] = make_uint4(gri[0], gri[1], gri[2], gri[3]);
      continue;
    }
    uint32_t pr[4], gr[4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
      // P^T: B[k = t][n = pole 8nb + gg] = p q^(15 - t);  b0: t = 2qq, 2qq+1;  b1: t = 2qq+8, 2qq+9
      const int n = 8 * nb + gg;
      float pn = 0.f, lq = 0.f;
      bool qpos = false;
      if (d < a.D && n < a.N) {
        pn = __ldg(a.p + (size_t)d * a.N + n);
        const float qn = __ldg(a.q + (size_t)d * a.N + n);
        qpos = qn > 0.f;
        lq = qpos ? __logf(qn) : 0.f;
      }
      pr[nb * 2 + 0] = bf16_bits(pn * qpow(lq, qpos, 15 - 2 * qq)) | (bf16_bits(pn * qpow(lq, qpos, 14 - 2 * qq)) << 16);
      pr[nb * 2 + 1] = bf16_bits(pn * qpow(lq, qpos, 7 - 2 * qq)) | (bf16_bits(pn * qpow(lq, qpos, 6 - 2 * qq)) << 16);
      // G^T: B[k = pole][n = t' = 8nb + gg] = g q^(t' + 1);  b0: poles 2qq, 2qq+1;  b1: poles 2qq+8, 2qq+9
      const int tp = 8 * nb + gg;
      float gv[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int pole = 2 * qq + (k & 1) + ((k >> 1) << 3);
        float v = 0.f;
        if (d < a.D && pole < a.N) {
          const float qn = __ldg(a.q + (size_t)d * a.N + pole);
          const bool qp = qn > 0.f;
          v = __ldg(a.g + (size_t)d * a.N + pole) * qpow(qp ? __logf(qn) : 0.f, qp, tp + 1);
        }
        gv[k] = v;
      }
      gr[nb * 2 + 0] = bf16_bits(gv[0]) | (bf16_bits(gv[1]) << 16);
      gr[nb * 2 + 1] = bf16_bits(gv[2]) | (bf16_bits(gv[3]) << 16);
    }
    Pc[ch * 32 + ln] = make_uint4(pr[0], pr[1], pr[2], pr[3]);
    Gc[ch * 32 + ln] = make_uint4(gr[0], gr[1], gr[2], gr[3]);
  }
  if (kPs && seg > 0 && tid == 0) {
    // the item of the run before (same tile and sequences) has written its statistics and states
    const int* flag = a.sched + 1 + ((int)ld_volatile_s(item_s) - a.n_items / a.n_seg);
    const long long start = clock64();
    const int* gave_up = a.sched + 1 + a.n_items;   // set by a CTA of this launch whose wait ran out
    for (;;) {
      int v;
      asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v != 0) break;
      if (*reinterpret_cast<const volatile int*>(gave_up) != 0) {  // the run before will never finish
        st_volatile_s(abort_s, 1u);
        break;
      }
      if (clock64() - start > wait_limit) {
        g_device_error = 3;
        st_volatile_s(abort_s, 1u);
        break;
      }
      __nanosleep(100);
    }
  }
  if constexpr (kPs) __syncthreads();   // the hand-off of the run before may be read

  if constexpr (kPs == 2) {
    // builder: the image of the matrices goes to global memory, and that is all
    __syncthreads();
    uint4* dst = reinterpret_cast<uint4*>(a.matrices + (size_t)blockIdx.x * kMatBytes);
    const uint4* src = reinterpret_cast<const uint4*>(sm + kOffT);
    for (int it = tid; it < kMatBytes / 16; it += kThreads) dst[it] = src[it];
    return;
  }
  if constexpr (kPs == 1) {
    if (!mbar_wait_lim(&xfree[0], 0u, abort_s, wait_limit)) { /* abort word set: every warp leaves at its first step */ }
  }
  // ---- running state of this thread: sequence b0 + g, channels 8*warp + e ----------------------
  const int bseq = b0 + g;
  const bool seq_ok = bseq < a.B;
  // kWp == 1: the running quantities live in registers from step to step.  kWp > 1: they arrive
  // through the mailbox at every step; a warp only keeps its latest mean per channel (mu_run), the
  // centre of its next sums of squares.
  float hc[kE][4];   // pole states: poles 2q, 2q+1, 8+2q, 9+2q of channel e
  float hci[kCplx ? kE : 1][4];  // kCplx: their imaginary parts
  float mu_run[kE], m2_run[kE], s1_run[kE];  // running mean, sum of squared deviations, sum of x
  float nbase = 1.f;
  const int cbase = warp * 8 + hf * kE;  // first channel of this warp inside the tile
  static_for<kE>([&](auto e_c) {
    constexpr int e = decltype(e_c)::value;
    const int d = d0 + cbase + e;
    const bool ok = seq_ok && d < a.D;
    if constexpr (kMail) {
      mu_run[e] = (kNorm && ok) ? a.prev_mean[(size_t)bseq * a.D + d] : 0.f;
      // The warps of the last group put the call's initial statistics and pole states into their
      // mailboxes, where step 0 (first group) looks for what "step -1" left (it does not wait: the
      // barrier before the loop orders these writes).
      if (kSm || wp == kWp - 1) {
        float c0 = 0.f, vv = 0.f;
        if (kNorm && ok) {
          c0 = (float)a.prev_count[bseq];
          vv = a.prev_var[(size_t)bseq * a.D + d];
        }
        sts128<e * 512>(mail_out, make_uint4(__float_as_uint(c0 * mu_run[e]), __float_as_uint(c0 * vv),
                                             __float_as_uint(mu_run[e]), 0u));
        float h4[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int pole = 2 * q + (k & 1) + ((k >> 1) << 3);
          h4[k] = (ok && a.h_in && pole < a.N) ? __ldg(a.h_in + ((size_t)bseq * a.D + d) * a.N + pole) : 0.f;
        }
        sts128<(kE + e) * 512>(mail_out, make_uint4(__float_as_uint(h4[0]), __float_as_uint(h4[1]),
                                                    __float_as_uint(h4[2]), __float_as_uint(h4[3])));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int pole = 2 * q + (k & 1) + ((k >> 1) << 3);
        if (kCplx) {
          const bool have = ok && a.h_in && pole < a.N;
          const size_t c = (((size_t)bseq * a.D + d) * a.N + pole) * 2;
          hc[e][k] = have ? __ldg(a.h_in + c) : 0.f;
          hci[e][k] = have ? __ldg(a.h_in + c + 1) : 0.f;
        } else if (kPs && kEma && seg > 0) {  // what the run before left (written by another SM: read past the L1)
          const float* hand = a.h_out ? a.h_out : a.handoff_h;
          hc[e][k] = (ok && pole < a.N) ? __ldcg(hand + ((size_t)bseq * a.D + d) * a.N + pole) : 0.f;
        } else {
          hc[e][k] = (kEma && ok && a.h_in && pole < a.N) ? __ldg(a.h_in + ((size_t)bseq * a.D + d) * a.N + pole) : 0.f;
        }
      }
      mu_run[e] = 0.f;
      m2_run[e] = 0.f;
      s1_run[e] = 0.f;
      if (kNorm && ok) {
        if (kPs && seg > 0) {
          // the running sums as the run before held them (bit for bit, so that the result does not
          // depend on the number of runs), its mean from the call's own output
          const float2 sm2 = __ldcg(reinterpret_cast<const float2*>(a.handoff_s) + (size_t)bseq * a.D + d);
          mu_run[e] = __ldcg(a.mean_out + (size_t)bseq * a.D + d);
          s1_run[e] = sm2.x;
          m2_run[e] = sm2.y;
        } else {
          const float c0 = (float)a.prev_count[bseq];
          const float mu = a.prev_mean[(size_t)bseq * a.D + d], vv = a.prev_var[(size_t)bseq * a.D + d];
          mu_run[e] = mu;
          m2_run[e] = c0 * vv;
          s1_run[e] = c0 * mu;
        }
      }
    }
  });
  if (kNorm && seq_ok) nbase = (float)a.prev_count[bseq] + 1.f;
  // kMask: running count of unmasked positions (exact in fp32: L < 2^24) and the mask row of this
  // thread's sequence; the flags of a step are fetched one step ahead
  float n_run = nbase - 1.f, nvalid = 0.f;
  const unsigned char* mrow = (kMask && seq_ok) ? a.mask + (size_t)bseq * L : nullptr;
  // (minus the 0/1 triangle: the prefix sums come out negated, which lets the finishing arithmetic
  // below form -(mean - c) and -(variance) with fused multiply-adds only)
  const float ut0 = (2 * q <= g) ? -1.f : 0.f, ut1 = (2 * q + 1 <= g) ? -1.f : 0.f;
  const float eps = a.eps;
  // position offsets of the 8 vectors this thread touches: j = 0..3 chunk 0, j = 4..7 chunk 1.
  // Rows of sequences g and g + 1 lie a multiple of 128 bytes apart, so the two sequences of a
  // quarter warp would hit the same banks: lanes with odd g therefore access the two positions of
  // each pair (t, t + 1) in the other order (slot j holds logical vector j ^ 1 there).
  // (Both LSU savings, this one and the all-ones MMAs below, are for the two-warps-per-column form;
  // with one warp per column the kernel is latency-bound and they cost 1 % instead.)
  constexpr bool kLeanLsu = kWs > 1;
  const bool odd = kLeanLsu && (g & 1) != 0;
  int toff[8];   // logical: vector j is position toff[j]
#pragma unroll
  for (int j = 0; j < 8; ++j) toff[j] = (j >> 2) * 16 + 2 * q + (j & 1) + ((j >> 1) & 1) * 8;
  // Tile addresses: slot j touches position 2q + p + 8 * ((j >> 1) & 1) + 16 * (j >> 2) with
  // p = (j & 1) ^ odd.  The 128-byte swizzle only looks at the position modulo 8, i.e. at 2q + p, so
  // two per-thread offsets (p = 0, 1) and compile-time immediates address all eight slots.
  constexpr int kRowB = kCg == 8 ? 128 : kCg * 16;
  uint32_t tb[2];
#pragma unroll
  for (int pq = 0; pq < 2; ++pq)
    tb[pq] = vec_off<kCg>(g, 2 * q + pq, warp) + (kWs == 2 ? hf * 8 : 0);
  const uint32_t tb0 = odd ? tb[1] : tb[0], tb1 = odd ? tb[0] : tb[1];  // slots with even / odd j
  // base addresses of the per-channel arrays (channel e of this warp adds a compile-time multiple)
  const uint32_t t_base = sm_s + kOffT + (cbase * 64 + lane) * 4;
  const uint32_t p_base = sm_s + kOffP + (cbase * kCm * 32 + lane) * 16;
  const uint32_t g_base = sm_s + kOffG + (cbase * kCm * 32 + lane) * 16;
  const uint32_t a_base = sm_s + kOffA + (cbase * 16 + 2 * q) * 4 * kCm;
  const uint32_t wb_base = sm_s + kOffWB + cbase * 16;

  __syncthreads();  // matrices visible

  // bit j: position toff[j] of step `step` is a valid (unmasked, in-range) position of this sequence
  auto mask_bits = [&](int step) -> uint32_t {
    uint32_t bits = 0;
    if (kMask && mrow != nullptr && step < nsteps) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int t = step * kStep + toff[j];
        const unsigned char m = t < L ? __ldg(mrow + t) : (unsigned char)1;
        bits |= (m == 0 ? 1u : 0u) << j;
      }
    }
    return bits;
  };
  uint32_t mk_next = mask_bits(wp);
  bool live = true;  // false once a bounded wait of this thread gave up
  for (int i = i_begin + wp; i < (kPs ? (int)ld_volatile_s(iend_s) : nsteps); i += kWp) {
    const int gi = kPs ? i + (int)ld_volatile_s(delta_s) : i;  // position in the ring
    const int s = gi % kStages;
    const uint32_t ph = (uint32_t)((gi / kStages) & 1);
    unsigned char* stage = sm + kOffStages + s * kStageBytes;
    const uint32_t stage_s = sm_s + kOffStages + s * kStageBytes;
    if (ld_volatile_s(abort_s) != 0) live = false;  // another waiter of this CTA gave up: leave together
    if (!__all_sync(0xffffffffu, live)) break;
    const bool ok = mbar_wait_lim(&full[s], ph, abort_s, wait_limit);
    // kWp > 1, first step of this warp (other than step 0): it has no mean of its own yet, so it
    // waits for the incoming statistics before it centres its sums (`early`)
    const bool early = kSm || (kWp > 1 && i < kWp);
    // phase of the hand-off barriers that the warp of step i - 1 completes with that step
    const uint32_t hand_par = kWp > 1 ? (uint32_t)((((i > 0 ? i - 1 : 0) / kWp)) & 1) : 0u;
    const uint32_t st0 = stage_s + tb0, st1 = stage_s + tb1;
    uint32_t v[8][kVw];
    static_for<8>([&](auto j_c) {
      constexpr int j = decltype(j_c)::value;
      constexpr int joff = (((j >> 1) & 1) * 8 + (j >> 2) * 16) * kRowB;
      if (kWs == 1) {
        const uint4 t4 = lds128<joff>((j & 1) ? st1 : st0);
        v[j][0] = t4.x; v[j][1] = t4.y; v[j][kVw - 2] = t4.z; v[j][kVw - 1] = t4.w;
      } else {
        const uint2 t2 = lds64<joff>((j & 1) ? st1 : st0);
        v[j][0] = t2.x; v[j][1] = t2.y;
      }
    });
    float invn[8];
    float inv_end = 0.f, n_end = 1.f, n_in = 0.f;
    const bool tail = !kMask && (i + 1) * kStep > L;
    uint32_t vm[kMask ? 8 : 1];   // all ones / zero per position: valid flag as an AND mask
    f32x2 vf2[kMask ? 4 : 1];     // the same as 1.0 / 0.0, position pairs
    bool step_has_valid = true;
    if constexpr (kMask) {
      const uint32_t cur = mk_next;
      mk_next = mask_bits(i + kWp);
      float vf[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vm[j] = 0u - ((cur >> j) & 1u);
        vf[j] = __uint_as_float(vm[j] & 0x3f800000u);
      }
      if constexpr (kNorm) {
#pragma unroll
      for (int jp = 0; jp < 4; ++jp) vf2[jp] = pack2(vf[2 * jp], vf[2 * jp + 1]);
      // prefix counts of the valid flags inside the halves, totals from the lane with q = 3
      float D0[4], D1[4];
      mma_tf32(D0, vf[0], vf[4], vf[1], vf[5], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
      mma_tf32(D1, vf[2], vf[6], vf[3], vf[7], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
      const int src3 = lane | 3;
      const float t0 = __shfl_sync(0xffffffffu, D0[1], src3), t1 = __shfl_sync(0xffffffffu, D1[1], src3);
      const float t2 = __shfl_sync(0xffffffffu, D0[3], src3), t3 = __shfl_sync(0xffffffffu, D1[3], src3);
      const float c0 = n_run, c1 = c0 - t0, c2 = c1 - t1, c3 = c2 - t2;   // (the triangle is negated)
      n_in = n_run;
      n_end = c3 - t3;
      const float cnt[8] = {c0 - D0[0], c0 - D0[1], c1 - D1[0], c1 - D1[1], c2 - D0[2], c2 - D0[3], c3 - D1[2], c3 - D1[3]};
#pragma unroll
      for (int j = 0; j < 8; ++j) invn[j] = rcp_fast(fmaxf(cnt[j], 1.f));
      step_has_valid = n_end > n_in;
      inv_end = rcp_fast(fmaxf(n_end, 1.f));
      nvalid += n_end - n_in;
      n_run = n_end;
      }
    } else if (kNorm) {
      const float nb_f = nbase + (float)(i * kStep);
#pragma unroll
      for (int j = 0; j < 8; ++j) invn[j] = rcp_fast(nb_f + (float)toff[j]);
      n_in = nb_f - 1.f;                                      // count before this step
      n_end = n_in + (float)min(kStep, L - i * kStep);        // count after this step
      inv_end = rcp_fast(n_end);
    }
    uint32_t vx[kXn ? 8 : 1][kXn ? kVw : 1];  // kXn: words of the normalised tile
    static_for<kVw>([&](auto pp_c) {
      constexpr int pp = decltype(pp_c)::value;
      float yv[2][8];
      float xq[kXn ? 2 : 1][8];
      static_for<2>([&](auto h2_c) {
        constexpr int h2 = decltype(h2_c)::value;
        constexpr int e = 2 * pp + h2;
        float xf[8];
        [[maybe_unused]] float xpad[(kMask && !kNorm) ? 8 : 1];   // the input at padded positions, 0 elsewhere
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          uint32_t w32 = odd ? v[j ^ 1][pp] : v[j][pp];
          if constexpr (kMask && !kNorm) {  // the EMA alone: omega multiplies the UNMASKED input
            const uint32_t pad = w32 & ~vm[j];
            xpad[j] = __uint_as_float(h2 == 0 ? (pad << 16) : (pad & 0xffff0000u));
          }
          if constexpr (kMask) w32 &= vm[j];   // a padded position enters every sum as 0
          xf[j] = __uint_as_float(h2 == 0 ? (w32 << 16) : (w32 & 0xffff0000u));
        }
        float xn[8];
        if (kNorm) {
          // kWp > 1: the statistics entering this step (sum of x, squared deviations about their
          // mean, that mean) come from the call's arguments at step 0 and from the mailbox of the
          // warp one step ahead otherwise
          float s1_in = 0.f, m2_in = 0.f, mean_in = 0.f;
          auto fetch_stats = [&]() {  // (step 0 finds the call's initial statistics in the mailbox)
            if (kLate && i != 0 && !mbar_try_s<e * 8>(flag_in, hand_par)) {
              if (!mbar_wait_slow(flag_in + e * 8, hand_par, abort_s, wait_limit)) live = false;
            }
            const uint4 m = lds128<e * 512>(mail_in);
            s1_in = __uint_as_float(m.x);
            m2_in = __uint_as_float(m.y);
            mean_in = __uint_as_float(m.z);
          };
          float cm = mu_run[e];
          if constexpr (kMail) {
            if (early) {
              fetch_stats();
              cm = mean_in;
            }
          }
          float S1[8], S2[8];
          float tot1, tot2;
          // Prefix sums inside each half (8 positions) of the two chunks: one tf32 MMA against the
          // 0/1 upper-triangular matrix per half.  The total of a half is its last prefix, held
          // by the lane with q = 3; a shuffle hands it to the row's other lanes, and the carries
          // (running total + totals of the halves before) are added afterwards in fp32.
          // All sums below are NEGATED (S1, S2, k1, k2, the E totals): the MMAs multiply by minus the
          // triangle, and the carries start from minus the running totals.
          float k1[4];  // carry of the sum of x for (row g, first half), (g, second), (g + 8, first), (g + 8, second)
          {  // sum of x: exact (bf16 inputs, fp32 accumulation)
            float D0[4], D1[4], E0[4], E1[4];
            mma_tf32(D0, xf[0], xf[4], xf[1], xf[5], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
            mma_tf32(D1, xf[2], xf[6], xf[3], xf[7], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
            // totals of the halves: the same rows against an all-ones matrix put the total into every
            // column, i.e. into every lane of the row (a shuffle goes through the LSU data pipe, which
            // the two-warps-per-column form loads to 60 %)
            if (kLeanLsu) {
              mma_tf32(E0, xf[0], xf[4], xf[1], xf[5], -1.f, -1.f, 0.f, 0.f, 0.f, 0.f);
              mma_tf32(E1, xf[2], xf[6], xf[3], xf[7], -1.f, -1.f, 0.f, 0.f, 0.f, 0.f);
            } else {  // the total of a half is its last prefix, held by the lane with q = 3
              const int src3 = lane | 3;
              E0[0] = __shfl_sync(0xffffffffu, D0[1], src3); E1[0] = __shfl_sync(0xffffffffu, D1[1], src3);
              E0[2] = __shfl_sync(0xffffffffu, D0[3], src3); E1[2] = __shfl_sync(0xffffffffu, D1[3], src3);
            }
            // kWp > 1: offsets of the halves only; the running total is added once it has arrived
            k1[0] = kLate ? 0.f : -(kSm ? s1_in : s1_run[e]);
            k1[1] = k1[0] + E0[0];
            k1[2] = k1[1] + E1[0];
            k1[3] = k1[2] + E0[2];
            tot1 = -k1[3] - E1[2];   // (positive; kLate: still without the incoming total)
            S1[0] = D0[0]; S1[1] = D0[1]; S1[4] = D0[2]; S1[5] = D0[3];
            S1[2] = D1[0]; S1[3] = D1[1]; S1[6] = D1[2]; S1[7] = D1[3];
          }
          // deviations from the centre, two positions (t, t + 1 of one row) per packed operation
          f32x2 dv2[4];
          const f32x2 cm2 = pack2(cm, cm);
          {
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
              dv2[jp] = sub2(pack2(xf[2 * jp], xf[2 * jp + 1]), cm2);
              if constexpr (kMask) dv2[jp] = mul2(dv2[jp], vf2[jp]);   // no deviation at a padded position
            }
          }
          float k2[4];  // the same carries for the sum of squared deviations
          {  // sum of (x - c)^2
            float sq[8];
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
              float lo, hi;
              unpack2(dv2[jp], lo, hi);
              sq[2 * jp] = lo * lo;
              sq[2 * jp + 1] = hi * hi;
            }
            float D0[4], D1[4], E0[4], E1[4];
            mma_tf32(D0, sq[0], sq[4], sq[1], sq[5], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
            mma_tf32(D1, sq[2], sq[6], sq[3], sq[7], ut0, ut1, 0.f, 0.f, 0.f, 0.f);
            if (kLeanLsu) {
              mma_tf32(E0, sq[0], sq[4], sq[1], sq[5], -1.f, -1.f, 0.f, 0.f, 0.f, 0.f);
              mma_tf32(E1, sq[2], sq[6], sq[3], sq[7], -1.f, -1.f, 0.f, 0.f, 0.f, 0.f);
            } else {
              const int src3 = lane | 3;
              E0[0] = __shfl_sync(0xffffffffu, D0[1], src3); E1[0] = __shfl_sync(0xffffffffu, D1[1], src3);
              E0[2] = __shfl_sync(0xffffffffu, D0[3], src3); E1[2] = __shfl_sync(0xffffffffu, D1[3], src3);
            }
            const float ea = E0[0], fa = E1[0], eb = E0[2], fb = E1[2];
            k2[0] = kLate ? 0.f : -(kSm ? m2_in : m2_run[e]);
            k2[1] = k2[0] + ea;
            k2[2] = k2[1] + fa;
            k2[3] = k2[2] + eb;
            tot2 = -(ea + fa) - (eb + fb);   // (positive)
            S2[0] = D0[0]; S2[1] = D0[1]; S2[4] = D0[2]; S2[5] = D0[3];
            S2[2] = D1[0]; S2[3] = D1[1]; S2[6] = D1[2]; S2[7] = D1[3];
          }
          if (tail) {
            // positions past the end hold x = 0, i.e. d = -c: take their squares (as the MMA saw
            // them, truncated to tf32) back out of the step total
            const float c2 = __uint_as_float(__float_as_uint(cm * cm) & 0xffffe000u);
            tot2 -= (float)(kStep - (L - i * kStep)) * c2;
          }
          // running totals entering the step; the incoming squared deviations are about the
          // incoming mean and move to this step's centre (sum (x-c)^2 = sum (x-m)^2 + n (m-c)^2)
          float m2_base;
          if constexpr (kSm) {
            m2_base = m2_in;   // (fetched before the sums; the centre is the incoming mean itself)
          } else if constexpr (kLate) {
            if (!early) fetch_stats();
            const float dm = mean_in - cm;
            m2_base = fmaf(n_in * dm, dm, m2_in);
            tot1 += s1_in;
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
              k1[jp] -= s1_in;
              k2[jp] -= m2_base;
            }
          } else {
            m2_base = m2_run[e];
          }
          // running statistics after this step: the new mean, and the squared deviations moved
          // from the centre c to it
          float mnew = tot1 * inv_end;
          const float shift = mnew - cm;
          float m2new = fmaf(-shift * shift, n_end, m2_base + tot2);
          if constexpr (kMask) {  // a step without a valid position leaves the statistics as they were
            mnew = step_has_valid ? mnew : cm;
            m2new = step_has_valid ? m2new : m2_base;
          }
          mu_run[e] = mnew;
          if constexpr (kMail) {
            sts128<e * 512>(mail_out, make_uint4(__float_as_uint(tot1), __float_as_uint(m2new), __float_as_uint(mnew), 0u));
            if constexpr (kLate) mbar_arrive_s<e * 8>(flag_out);
          } else {
            s1_run[e] = tot1;
            m2_run[e] = m2new;
          }
          const uint4 wbu = lds128<e * 16>(wb_base);   // {w, w, b, b}
          {
            const f32x2 neps2 = pack2(-eps, -eps);
            const f32x2 w2 = pack2(__uint_as_float(wbu.x), __uint_as_float(wbu.y));
            const f32x2 b2 = pack2(__uint_as_float(wbu.z), __uint_as_float(wbu.w));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {
              const f32x2 in2 = pack2(invn[2 * jp], invn[2 * jp + 1]);
              // (negated sums) nu = c - mean, ne = -(E[d^2] + eps), nv = nu^2 + ne = -(variance + eps)
              const f32x2 nu2 = fma2(add2(pack2(S1[2 * jp], S1[2 * jp + 1]), pack2(k1[jp], k1[jp])), in2, cm2);
              const f32x2 ne2 = fma2(add2(pack2(S2[2 * jp], S2[2 * jp + 1]), pack2(k2[jp], k2[jp])), in2, neps2);
              float nva, nvb;
              unpack2(fma2(nu2, nu2, ne2), nva, nvb);
              const f32x2 sc2 = mul2(pack2(rsqrt_fast(fmaxf(-nva, eps)), rsqrt_fast(fmaxf(-nvb, eps))), w2);
              f32x2 xn2 = fma2(add2(dv2[jp], nu2), sc2, b2);
              if constexpr (kMask) xn2 = mul2(xn2, vf2[jp]);   // TimestepNorm writes 0 at a padded position
              unpack2(xn2, xn[2 * jp], xn[2 * jp + 1]);
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) xn[j] = xf[j];
        }
        if (kXn) {
#pragma unroll
          for (int j = 0; j < 8; ++j) xq[h2][j] = xn[j];
        }
        if (!kEma) {
#pragma unroll
          for (int j = 0; j < 8; ++j) yv[h2][j] = xn[j];
          return;
        }
        // A fragment of xn: a0 (row g: t = 2q, 2q+1), a1 (row g+8), a2 (row g: t = 2q+8, 2q+9), a3 (row g+8)
        const uint32_t xa0 = pack_bf16(xn[0], xn[1]), xa2 = pack_bf16(xn[2], xn[3]);
        const uint32_t xa1 = pack_bf16(xn[4], xn[5]), xa3 = pack_bf16(xn[6], xn[7]);
        const uint2 tr = make_uint2(lds32<e * 256>(t_base), lds32<e * 256 + 128>(t_base));
        float W0[4], W1[4];  // Toeplitz term of the outputs (positions 0..7 and 8..15 of each chunk)
        mma_bf16(W0, xa0, xa1, xa2, xa3, tr.x, 0u, 0.f, 0.f, 0.f, 0.f);
        mma_bf16(W1, xa0, xa1, xa2, xa3, tr.y, tr.x, 0.f, 0.f, 0.f, 0.f);
        float Y0[4], Y1[4];
        if (kCplx) {
          const uint4 prr = lds128<e * 1024>(p_base);
          const uint4 pri = lds128<e * 1024 + 512>(p_base);
          const uint4 grr = lds128<e * 1024>(g_base);
          const uint4 gri = lds128<e * 1024 + 512>(g_base);
          // q^16 of poles 2q, 2q+1 and 8+2q, 9+2q as (re, im) pairs
          const uint4 a0u = lds128<e * 128>(a_base);
          const uint4 a1u = lds128<e * 128 + 64>(a_base);
          const float ar[4] = {__uint_as_float(a0u.x), __uint_as_float(a0u.z), __uint_as_float(a1u.x), __uint_as_float(a1u.z)};
          const float ai[4] = {__uint_as_float(a0u.y), __uint_as_float(a0u.w), __uint_as_float(a1u.y), __uint_as_float(a1u.w)};
          float Hr0[4], Hr1[4], Hi0[4], Hi1[4];
          mma_bf16(Hr0, xa0, xa1, xa2, xa3, prr.x, prr.y, 0.f, 0.f, 0.f, 0.f);
          mma_bf16(Hr1, xa0, xa1, xa2, xa3, prr.z, prr.w, 0.f, 0.f, 0.f, 0.f);
          mma_bf16(Hi0, xa0, xa1, xa2, xa3, pri.x, pri.y, 0.f, 0.f, 0.f, 0.f);
          mma_bf16(Hi1, xa0, xa1, xa2, xa3, pri.z, pri.w, 0.f, 0.f, 0.f, 0.f);
          // local contributions per pole k: chunk 0 (row g) and chunk 1 (row g + 8)
          const float l0r[4] = {Hr0[0], Hr0[1], Hr1[0], Hr1[1]}, l0i[4] = {Hi0[0], Hi0[1], Hi1[0], Hi1[1]};
          const float l1r[4] = {Hr0[2], Hr0[3], Hr1[2], Hr1[3]}, l1i[4] = {Hi0[2], Hi0[3], Hi1[2], Hi1[3]};
          float s0r[4], s0i[4], s1r[4], s1i[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            s0r[k] = hc[e][k];
            s0i[k] = hci[e][k];
            s1r[k] = fmaf(ar[k], s0r[k], fmaf(-ai[k], s0i[k], l0r[k]));
            s1i[k] = fmaf(ar[k], s0i[k], fmaf(ai[k], s0r[k], l0i[k]));
            hc[e][k] = fmaf(ar[k], s1r[k], fmaf(-ai[k], s1i[k], l1r[k]));
            hci[e][k] = fmaf(ar[k], s1i[k], fmaf(ai[k], s1r[k], l1i[k]));
          }
          const uint32_t hr0 = pack_bf16(s0r[0], s0r[1]), hr1 = pack_bf16(s1r[0], s1r[1]);
          const uint32_t hr2 = pack_bf16(s0r[2], s0r[3]), hr3 = pack_bf16(s1r[2], s1r[3]);
          const uint32_t hi0 = pack_bf16(s0i[0], s0i[1]), hi1 = pack_bf16(s1i[0], s1i[1]);
          const uint32_t hi2 = pack_bf16(s0i[2], s0i[3]), hi3 = pack_bf16(s1i[2], s1i[3]);
          float Z0[4], Z1[4];
          mma_bf16(Z0, hr0, hr1, hr2, hr3, grr.x, grr.y, W0[0], W0[1], W0[2], W0[3]);
          mma_bf16(Z1, hr0, hr1, hr2, hr3, grr.z, grr.w, W1[0], W1[1], W1[2], W1[3]);
          mma_bf16(Y0, hi0, hi1, hi2, hi3, gri.x, gri.y, Z0[0], Z0[1], Z0[2], Z0[3]);
          mma_bf16(Y1, hi0, hi1, hi2, hi3, gri.z, gri.w, Z1[0], Z1[1], Z1[2], Z1[3]);
        } else {
          const uint4 pr = lds128<e * 512>(p_base);
          const uint4 gr = lds128<e * 512>(g_base);
          const uint2 aq0u = lds64<e * 64>(a_base);
          const uint2 aq1u = lds64<e * 64 + 32>(a_base);
          const float2 aq0 = make_float2(__uint_as_float(aq0u.x), __uint_as_float(aq0u.y));
          const float2 aq1 = make_float2(__uint_as_float(aq1u.x), __uint_as_float(aq1u.y));
          // local state contributions of the two chunks
          float H0[4], H1[4];
          mma_bf16(H0, xa0, xa1, xa2, xa3, pr.x, pr.y, 0.f, 0.f, 0.f, 0.f);  // poles 2q, 2q+1
          mma_bf16(H1, xa0, xa1, xa2, xa3, pr.z, pr.w, 0.f, 0.f, 0.f, 0.f);  // poles 8+2q, 9+2q
          // states entering chunk 0 (= carried) and chunk 1, and the new carry
          float hs0[4];
          if constexpr (kMail) {
            // pole states entering the step: from the mailbox of the warp one step ahead (step 0
            // finds the call's h_in there)
            if (kLate && i != 0 && !mbar_try_s<(kE + e) * 8>(flag_in, hand_par)) {
              if (!mbar_wait_slow(flag_in + (kE + e) * 8, hand_par, abort_s, wait_limit)) live = false;
            }
            const uint4 m = lds128<(kE + e) * 512>(mail_in);
            hs0[0] = __uint_as_float(m.x); hs0[1] = __uint_as_float(m.y);
            hs0[2] = __uint_as_float(m.z); hs0[3] = __uint_as_float(m.w);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) hs0[k] = hc[e][k];
          }
          float hs1[4], hn[4];
          hs1[0] = fmaf(aq0.x, hs0[0], H0[0]);
          hs1[1] = fmaf(aq0.y, hs0[1], H0[1]);
          hs1[2] = fmaf(aq1.x, hs0[2], H1[0]);
          hs1[3] = fmaf(aq1.y, hs0[3], H1[1]);
          hn[0] = fmaf(aq0.x, hs1[0], H0[2]);
          hn[1] = fmaf(aq0.y, hs1[1], H0[3]);
          hn[2] = fmaf(aq1.x, hs1[2], H1[2]);
          hn[3] = fmaf(aq1.y, hs1[3], H1[3]);
          if constexpr (kMail) {
            sts128<(kE + e) * 512>(mail_out, make_uint4(__float_as_uint(hn[0]), __float_as_uint(hn[1]),
                                                        __float_as_uint(hn[2]), __float_as_uint(hn[3])));
            if constexpr (kLate) mbar_arrive_s<(kE + e) * 8>(flag_out);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) hc[e][k] = hn[k];
          }
          const uint32_t ha0 = pack_bf16(hs0[0], hs0[1]), ha1 = pack_bf16(hs1[0], hs1[1]);
          const uint32_t ha2 = pack_bf16(hs0[2], hs0[3]), ha3 = pack_bf16(hs1[2], hs1[3]);
          // outputs: the carried-state term accumulates onto the Toeplitz term, which does not
          // wait for the states (W0, W1 are issued alongside H0, H1 above)
          mma_bf16(Y0, ha0, ha1, ha2, ha3, gr.x, gr.y, W0[0], W0[1], W0[2], W0[3]);
          mma_bf16(Y1, ha0, ha1, ha2, ha3, gr.z, gr.w, W1[0], W1[1], W1[2], W1[3]);
        }
        yv[h2][0] = Y0[0]; yv[h2][1] = Y0[1]; yv[h2][4] = Y0[2]; yv[h2][5] = Y0[3];
        yv[h2][2] = Y1[0]; yv[h2][3] = Y1[1]; yv[h2][6] = Y1[2]; yv[h2][7] = Y1[3];
        if constexpr (kMask && !kNorm) {
          // the Toeplitz diagonal carries omega times the masked input: a padded position still gets
          // omega times its own (unmasked) input, as the reference's residual does
          const float om = __uint_as_float(lds32<e * 16>(wb_base));
#pragma unroll
          for (int j = 0; j < 8; ++j) yv[h2][j] = fmaf(om, xpad[j], yv[h2][j]);
        }
        if (kSilu) {
#pragma unroll
          for (int j = 0; j < 8; ++j) yv[h2][j] = silu_tanh(yv[h2][j]);
        }
      });
#pragma unroll
      for (int j = 0; j < 8; j += 2) {
        const uint32_t o0 = pack_bf16(yv[0][j], yv[1][j]), o1 = pack_bf16(yv[0][j + 1], yv[1][j + 1]);
        v[j][pp] = odd ? o1 : o0;
        v[j + 1][pp] = odd ? o0 : o1;
        if (kXn) {
          const uint32_t n0 = pack_bf16(xq[0][j], xq[1][j]), n1 = pack_bf16(xq[0][j + 1], xq[1][j + 1]);
          vx[j][pp] = odd ? n1 : n0;
          vx[j + 1][pp] = odd ? n0 : n1;
        }
      }
    });
    if (kXn) {
      // the store that read this buffer two steps ago must have drained it
      if (i >= 2 && !mbar_wait_lim(&xfree[i & 1], (uint32_t)(((i >> 1) - 1) & 1), abort_s, wait_limit)) live = false;
      const uint32_t xb = sm_s + C::kOffXn + (i & 1) * kStageBytes;
      static_for<8>([&](auto j_c) {
        constexpr int j = decltype(j_c)::value;
        constexpr int joff = (((j >> 1) & 1) * 8 + (j >> 2) * 16) * kRowB;
        if (kWs == 1)
          sts128<joff>(xb + ((j & 1) ? tb1 : tb0), make_uint4(vx[j][0], vx[j][1], vx[j][kVw - 2], vx[j][kVw - 1]));
        else
          sts64<joff>(xb + ((j & 1) ? tb1 : tb0), make_uint2(vx[j][0], vx[j][1]));
      });
    }
    static_for<8>([&](auto j_c) {
      constexpr int j = decltype(j_c)::value;
      constexpr int joff = (((j >> 1) & 1) * 8 + (j >> 2) * 16) * kRowB;
      if (kWs == 1)
        sts128<joff>((j & 1) ? st1 : st0, make_uint4(v[j][0], v[j][1], v[j][kVw - 2], v[j][kVw - 1]));
      else
        sts64<joff>((j & 1) ? st1 : st0, make_uint2(v[j][0], v[j][1]));
    });
    fence_proxy_async();
    __syncwarp();
    // A wait that gave up (never expected) leaves the tile unfinished: nothing more is stored, and
    // every warp of the CTA leaves the loop at its next step (abort word).
    if (!ok) live = false;
    if (__all_sync(0xffffffffu, live)) {
      if (lane == 0) mbar_arrive(&done[s]);
      // warps run on to their next stage on their own; only the issuing thread of this group waits
      // for the whole tile
      if (issuer) {
        if (mbar_wait_lim(&done[s], ph, abort_s, wait_limit)) {
          tma_store_3d(&tmy, d0, i * kStep, b0, stage);
          if (kXn) tma_store_3d(&tmn, d0, i * kStep, b0, sm + C::kOffXn + (i & 1) * kStageBytes);
          bulk_commit();
          if (kXn) {
            bulk_wait_read<1>();  // the stores of the step before have drained their stage and buffer
            if (i >= 1) mbar_arrive(&xfree[(i - 1) & 1]);
          }
          // refill: the stage of this thread's previous store (step i - kWp) takes tile i - kWp + kStages
          const int nt = i + kStages - kWp;
          if (nt < (kPs ? (int)ld_volatile_s(iend_s) : nsteps)) {
            if (!kXn) bulk_wait_read<1>();  // the store issued before this one has drained its stage
            const int s2 = (kPs ? gi + kStages - kWp : nt) % kStages;
            mbar_expect_tx(&full[s2], kStageBytes);
            if (nt != a.withhold_step)
              tma_load_3d(sm + kOffStages + s2 * kStageBytes, &tmx, d0, nt * kStep, b0, &full[s2]);
          }
        } else {
          live = false;
        }
      }
    }
  }
  if (issuer) bulk_wait<0>();
  if (ld_volatile_s(abort_s) != 0) live = false;
  if (!live) {  // the error word is raised; the final statistics and states are not written
    // (segmented: the runs that depend on this one learn of it instead of waiting out their limits)
    if (kPs && lane == 0) *reinterpret_cast<volatile int*>(a.sched + 1 + a.n_items) = 1;
    return;
  }

  // ---- final statistics and states -------------------------------------------------------------
  if constexpr (kMail) {
    // held by the group of the last step, in its own mailbox
    if (kLate && wp != (nsteps - 1) % kWp) return;
    static_for<kE>([&](auto e_c) {
      constexpr int e = decltype(e_c)::value;
      if (kNorm) {
        const uint4 m = lds128<e * 512>(mail_out);
        m2_run[e] = __uint_as_float(m.y);
        mu_run[e] = __uint_as_float(m.z);
      }
      const uint4 hm = lds128<(kE + e) * 512>(mail_out);
      hc[e][0] = __uint_as_float(hm.x); hc[e][1] = __uint_as_float(hm.y);
      hc[e][2] = __uint_as_float(hm.z); hc[e][3] = __uint_as_float(hm.w);
    });
  }
  if (seq_ok && q == 0) {
#pragma unroll
    for (int e = 0; e < kE; ++e) {
      const int d = d0 + cbase + e;
      if (kNorm && d < a.D) {
        const int i_last = kPs ? (int)ld_volatile_s(iend_s) : nsteps;
        const float n = kMask ? n_run : (float)a.prev_count[bseq] + (float)min(i_last * kStep, L);
        float mo = mu_run[e], vo = fmaxf(m2_run[e] / n, 0.f);
        if (kMask && !(n > 0.f)) {  // nothing counted, before or in this call: the incoming statistics stand
          mo = a.prev_mean[(size_t)bseq * a.D + d];
          vo = a.prev_var[(size_t)bseq * a.D + d];
        }
        a.mean_out[(size_t)bseq * a.D + d] = mo;
        a.var_out[(size_t)bseq * a.D + d] = vo;
        if constexpr (kPs)
          reinterpret_cast<float2*>(a.handoff_s)[(size_t)bseq * a.D + d] = make_float2(s1_run[e], m2_run[e]);
      }
    }
    if (kNorm && d0 == 0 && (!kPs || (int)ld_volatile_s(iend_s) == nsteps) && warp == 0 && hf == 0)
      a.count_out[bseq] = a.prev_count[bseq] + (kMask ? (long long)nvalid : (long long)L);
  }
  // (kPs: a run that is not the last leaves its pole states for the next one, in h_out if the call has one)
  float* const h_dst = (kPs && !a.h_out && (int)ld_volatile_s(iend_s) < nsteps) ? a.handoff_h : a.h_out;
  if (kEma && seq_ok && h_dst) {
#pragma unroll
    for (int e = 0; e < kE; ++e) {
      const int d = d0 + cbase + e;
      if (d < a.D) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int pole = 2 * q + (k & 1) + ((k >> 1) << 3);
          if (pole < a.N) {
            if (kCplx) {
              const size_t c = (((size_t)bseq * a.D + d) * a.N + pole) * 2;
              h_dst[c] = hc[e][k];
              h_dst[c + 1] = hci[e][k];
            } else {
              h_dst[((size_t)bseq * a.D + d) * a.N + pole] = hc[e][k];
            }
          }
        }
      }
    }
  }
  if constexpr (kPs) {
    // publish: every thread's statistics and states are written, then the item's flag is set
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(a.sched + 1 + (int)ld_volatile_s(item_s)), "r"(1) : "memory");
    }
  }
}

// xn (with its strides nsb, nsl) is the optional second output; kXn selects the kernel form.
template <bool kNorm, int kCg, bool kSilu, int kWs = 1, bool kXn = false, bool kEma = true, bool kCplx = false,
          int kWp = 1, bool kMask = false, bool kSm = false>
static bool launch_variant(int dtype, const void* x, void* y, long long xsb, long long xsl, long long ysb,
                           long long ysl, const StreamArgs& a, cudaStream_t s, void* xn = nullptr,
                           long long nsb = 0, long long nsl = 0) {
  using C = Cfg<kCg, kXn, kCplx, kWs, kWp, kSm>;
  const CUtensorMapSwizzle sw = kCg == 8 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUtensorMap tx, ty, tn;
  if (!make_tensor_map_3d(&tx, dtype, x, a.D, a.L, a.B, xsl, xsb, C::kCh, kStep, kSeq, sw)) return false;
  if (!make_tensor_map_3d(&ty, dtype, y, a.D, a.L, a.B, ysl, ysb, C::kCh, kStep, kSeq, sw)) return false;
  if (kXn) {
    if (!make_tensor_map_3d(&tn, dtype, xn, a.D, a.L, a.B, nsl, nsb, C::kCh, kStep, kSeq, sw)) return false;
  } else {
    tn = ty;
  }
  auto kern = tsn_ema_mma_kernel<kNorm, kCg, kSilu, kWs, kXn, kEma, kCplx, kWp, kMask, kSm>;
  static std::once_flag once;
  static bool attr_ok = true;
  std::call_once(once, [&] {
    attr_ok = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) == cudaSuccess;
  });
  if (!attr_ok) {
    cudaGetLastError();
    return false;
  }
  dim3 grid((a.D + C::kCh - 1) / C::kCh, (a.B + kSeq - 1) / kSeq);
  launch(kern, grid, dim3(kCg * kWs * kWp * 32), (size_t)C::kSmemBytes, (void*)s, tx, ty, tn, a);
  static const std::string name = std::string("tsn_ema_mma tile=") + std::to_string(kCg) + " warps_per_column=" +
                                  std::to_string(kWs) + " pipe=" + std::to_string(kWp) + (kNorm ? " norm" : "") +
                                  (kEma ? " ema" : "") + (kCplx ? " complex" : "") + (kXn ? " xn" : "") + (kMask ? " mask" : "") + (kSm ? " smstate" : "");
  g_last_kernel.store(name.c_str(), std::memory_order_relaxed);
  return true;
}

}  // namespace

}  // namespace mega
