// tcgen05 kernel for the four walks of chunked retention on sm_100a (one template, four roles):
//   MODE_FWD, forward walk : outputs O (+ final state, + POP block states)   replaces fused_chunk_retention_fwd /
//                                                                            fused_pop_retention_fwd of the reference
//   MODE_DQ,  forward walk : dQ (recomputes the states)                      replaces fused_retention_bwd_dq
//   MODE_FWD, reverse walk : dV and dS_0, with (X, K, V) := (K, Q, dO)       replace fused_retention_bwd_dk_dv_ds /
//   MODE_DQ,  reverse walk : dK,          with (X, K, V) := (V, Q, dO)       pop_retention_bwd_dk_dv_ds
// The reverse walks carry G = d(loss)/d(state after the chunk) instead of the state and add the POP
// block-state gradients where a block ends (flash_pop/pop_retention/pop_bwd.py:137-159).  In a
// reverse walk the in-place row scale is zeta_i = gamma^(i+1) on dO, the mask is upper triangular and
// the output row scale is eta_j * rs:
//   dV_j = eta_j rs [ K Gb + triu(K Q^T) gamma^-L (zeta.dO) ]_j     dK_j = eta_j rs [ V Gb^T + triu(V (zeta.dO)^T) gamma^-L Q ]_j
//   G <- gamma^L G + Q^T (zeta.dO)                                  (flash_pop/fused_retention/fused_chunk_bwd.py:180-215)
//
// One CTA walks one (batch, head) sequence chunk by chunk (C = 64 tokens) for one tile of the state:
// R state rows (of dk) x CC state columns (of dv).  The fp32 state lives in the registers of the
// "state" warps for the whole sequence; HBM traffic is the activations in and the result out.
//
// Per chunk of L <= 64 tokens, gamma = head decay, rs = 1/sqrt(dk), X = Q (FWD) or dO (DQ):
//   Veta_j = gamma^(L-1-j) v_j                      scaled in place in shared memory (rows >= L zeroed)
//   Sc     = X K^T            (FWD)   |  X Veta^T   (DQ)             tcgen05, 64x64 fp32 in tensor memory
//   P'     = tril(Sc) * gamma^-L * rs  -> bf16      registers -> swizzled shared memory
//   ACC    = X Sb + P' Veta   (FWD)   |  X Sb^T + P' K   (DQ)        Sb = bf16 copy of the chunk-start state
//   out_i  = gamma^(i+1) * ACC_i                                      epilogue, TMA store
//   dS     = K^T Veta ;  S <- gamma^L S + rs dS                       state warps, fp32 registers
// which equals the reference's  O = (QK^T.D)V + zeta.(Q S),  S <- gamma^L S + (K.eta)^T V
// (flash_pop/fused_retention/fused_chunk_fwd.py:35-52,75-90) because gamma^(i-j) =
// gamma^(i+1) * gamma^-L * gamma^(L-1-j): the decay mask factors into a row scale, a constant and
// the column scale already folded into Veta, so no [C,C] mask table is needed.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer, warps 2-5 "score" warps (P', output epilogue),
// warps 6.. "state" warps (in-place row scaling of V, state update, bf16 state copy), and in the 128-wide tiles two
// more MMA-issuing warps after them (Cfg::NMMA).  All hand-offs are mbarriers; every wait is bounded and reports
// through the status word instead of hanging.
//
// Scheduling.  Per chunk the work is a feed-forward chain (TMA -> V scaling -> Sc, dS -> P', state update
// -> X Sb, P' V -> epilogue) whose every hand-off costs a few hundred cycles; only the fp32 state
// recurrence in the state warps' registers is truly serial.  So no role walks the chunks in lock step:
// the state warps and the score warps (and the MMA issuer where it is one warp) each POLL their input barriers and run
// whichever of their tasks is ready (scores of chunk n+1 before the products of chunk n if that is what has arrived),
// with the score tile, P' and the accumulator double-buffered where tensor/shared memory allows, so that
// several chunks are in flight per SM and the chain latency is hidden.
//
// Output.  Each score warp owns 16 rows of an accumulator and stores them itself: through its slice of a staging
// tile and a 16-row TMA store (tiles wider than 64 columns), or straight from tensor memory to global memory
// (64-column tiles).  No barrier joins the score warps.
//
// Under-filled launches.  When batch x heads x tiles covers less than half of the GPU, the launcher cuts every sequence
// into T-segments (segment_scan.cu): a STATE_ONLY instance of this kernel computes each segment's local end state
// (increments only, no scores, no output), a small scan turns those into the segments' start states, and the walk
// proper then runs one CTA per (batch, head, tile, segment) from its start state in fp32 scratch memory.
//
// Suffix calls (thousands of sequences of a few chunks, each starting from its own state and dropping its end
// state) may be regrouped by the launcher: G consecutive suffixes of a row as one sequence of G*T tokens with block
// size T, the state replaced at every suffix start - same results, one CTA set-up per G suffixes.
//
// dv = 256 beside dk = 128.  A MODE_DQ walk may cut dv instead of dk (ScanParams::col_split): two CTAs per head on the
// 128 x 128 instance, each with its half of the state columns; its output tile is then a partial sum, which the TMA
// unit adds to the zeroed output (cp.reduce.async.bulk.tensor, performed in L2).
#include <atomic>
#include <cmath>
#include <type_traits>

#include "fpb_common.cuh"
#include "ptx_sm100.cuh"
#include "scan_common.cuh"
#include "tensormap.cuh"
#include "umma_launch.h"

namespace fpb {
namespace {

using namespace ptx;
using namespace scan;
typedef __nv_bfloat16 bf16;

// The tcgen05.mma issue loops (4-8 k-steps each) are fully unrolled: rolled loops measured slower at d = 128.
#define FPB_UNROLL_MMA _Pragma("unroll")

constexpr int MODE_FWD = 0, MODE_DQ = 1;
constexpr int SCORE_WARP0 = 2, STATE_WARP0 = 6;
constexpr int N_SCORE = 128;


struct ScanParams {
  CUtensorMap map_x, map_k, map_v, map_out;   // map_out: 16-row boxes
  bf16* out; int64_t out_sb, out_st, out_sh;
  // states are bf16 or fp32 (state_f32), strides in elements
  const void* s0; int64_t s0_sb, s0_sh;
  void* s_out; int64_t so_sb, so_sh;
  void* block_states;            // forward walk: states after full blocks (written)
  const void* block_grads;       // reverse walk: gradients of those states (read)
  void* sfx_blocks; int32_t sfx_M, sfx_N;   // suffix calls: start states (forward) / their gradients (reverse)
  int32_t sfx_G;                 // suffixes walked back to back by one CTA as one sequence of sfx_G * block_size tokens (>= 1)
  int32_t T, H, dk, dv, block_size, n_blocks;
  int32_t sched_bs;              // block size the chunk schedule is cut at: block_size, or 0 when block states are
                                 // emitted from inside full chunks (forward walk, 64 x 64 tiles, see EMIT below)
  int32_t state_f32;             // element type of s0, s_out, block states / gradients and suffix start states
  int32_t col_split;             // MODE_DQ walks only: the tiles cut dv (columns of the state) instead of dk, so each CTA's
                                 // output tile is a partial sum over its dv columns; TMA adds it to `out` (zeroed before)
  int32_t n_seg, seg_len;        // T-segments: blockIdx.z = batch * n_seg + segment, segment s covers tokens [s * seg_len, ...)
  float* seg_states;             // fp32 (B, H, n_seg, dk, dv): start values of the segments (local end values in a STATE_ONLY pass)
  WalkTuning tune;
  int32_t* status;
  long long* trace;              // diagnostics: per-chunk clock64() stamps of CTA (0,0,0), or null
  float log2g[FPB_MAX_HEADS];
};

// barrier slots (8 bytes each) at the start of the barrier page - three per stage of the tile ring, then the fixed
// ones - then two 4-byte words and the wait limit
constexpr int MAXS = 6;          // most stages a configuration may have
enum { B_FULL = 0, B_EMPTY = MAXS, B_VRDY = 2 * MAXS, B_SCFULL = 3 * MAXS, B_PRDY = B_SCFULL + 2, B_ACCFULL = B_PRDY + 2,
       B_ACCFREE = B_ACCFULL + 2, B_DSFULL = B_ACCFREE + 2, B_DSFREE = B_DSFULL + 2, B_SBRDY = B_DSFREE + 2, B_SBFREE = B_SBRDY + 2,
       B_DSPFULL = B_SBFREE + 2, B_DSPFREE = B_DSPFULL + 1, B_COUNT = B_DSPFREE + 1 };
constexpr int OFF_TMEM_SLOT = B_COUNT * 8, OFF_ABORT = OFF_TMEM_SLOT + 4, OFF_LIMIT = OFF_ABORT + 4, BAR_PAGE = 512;
static_assert(OFF_LIMIT % 8 == 0 && OFF_LIMIT + 8 <= BAR_PAGE, "the wait limit sits right after the abort flag");

// DEEP: a variant of the small-tile configurations for launches of at most one CTA per SM.  The small tiles normally
// run two CTAs per SM with the three stages each half of the shared memory holds; a lone CTA on its SM is then bound by
// how many chunks it can have in flight (a chunk holds its stage for about 12 k cycles from the issue of its copies to
// the completion of its last product), so the lone CTA takes the whole shared memory: six stages, two P' buffers.
template <int MODE, int R, int CC, bool DEEP = false>
struct Cfg {
  static constexpr int W1 = MODE == MODE_FWD ? R : CC;       // width of X (and of the Sc contraction)
  static constexpr int NOUT = MODE == MODE_FWD ? CC : R;     // width of the output tile
  // Output rows go from tensor memory through registers straight to global memory (measured faster for 64-wide
  // output tiles) or through a staging tile and a TMA store (faster for the wider ones).
  static constexpr bool DIRECT_OUT = NOUT == 64;
  // one CTA per SM for the large state tiles (128x128, 64x256), two for the small ones
  static constexpr bool ONE = R * CC >= 128 * 128;
  static constexpr bool SOLO = ONE || DEEP;                  // one CTA per SM
  // state warps: their three tasks per chunk are latency, not instructions, so a CTA that has its SM to itself spreads
  // the state over eight warps (the deep 64 x 64 variant: forward -8 %, dQ walk -13 % against four; sixteen: +4 %)
  static constexpr int STATE_WARPS = (ONE || DEEP) ? 8 : 4;
  static constexpr int N_STATE = 32 * STATE_WARPS;
  // The 128-wide one-CTA-per-SM configurations issue their products from THREE warps, one per chain of products, each a
  // plain loop over the chunks that blocks on the barriers of its next product: scores | increment | state term, then
  // intra-chunk term (same accumulator, in that order).  One warp polling for whichever product is ready - about 3000
  // cycles of barrier tests, descriptor arithmetic, tcgen05.mma and commits per chunk - was the walk's pacemaker; two
  // polling warps gained 5-6 %, three blocking ones another 2-3 %.  (The deep 64 x 64 variant gains nothing from either.)
  static constexpr int NMMA = ONE ? 3 : 1;
  static constexpr int MMAB_WARP = STATE_WARP0 + STATE_WARPS;
  static constexpr int MMAC_WARP = MMAB_WARP + 1;
  static constexpr int NTHREADS = STATE_WARP0 * 32 + N_STATE + (NMMA - 1) * 32;
  static constexpr int MIN_CTAS = SOLO ? 1 : 2;
  static constexpr int NP = SOLO ? 2 : 1;                    // P' buffers
  static constexpr int X_BYTES = C * W1 * 2, K_BYTES = C * R * 2, V_BYTES = C * CC * 2;
  static constexpr int STAGE_BYTES = X_BYTES + K_BYTES + V_BYTES;
  static constexpr int P_BYTES = C * C * 2;
  static constexpr int SB_BYTES = R * CC * 2;
  // bf16 copies of the state.  Two (so that the copy for chunk n + 1 need not wait for the state-term product of chunk
  // n to finish reading) measured no gain next to the small tiles, and next to the 128 x 128 tile - where the second
  // copy takes the place of the output staging tile - a loss of 3 % on top of the 8 % the direct epilogue costs: one.
  static constexpr int NSB = 1;
  static constexpr int OUT_BYTES = C * NOUT * 2;
  static constexpr int FIXED = NP * P_BYTES + NSB * SB_BYTES + OUT_BYTES + BAR_PAGE;
  static constexpr int SMEM_LIMIT = SOLO ? 226 * 1024 : 115712;  // (233472 B per SM) / 2 - 1 KB system reserve
  static constexpr int FIT = (SMEM_LIMIT - FIXED) / STAGE_BYTES;
  static constexpr int STAGES = DEEP ? (FIT < MAXS ? FIT : MAXS) : (FIT >= 3 ? 3 : 2);
  static_assert(STAGES >= 2, "at least two stages");
  static constexpr int OFF_STAGE = 0;
  static constexpr int OFF_P = STAGES * STAGE_BYTES;
  static constexpr int OFF_SB = OFF_P + NP * P_BYTES;
  static constexpr int OFF_OUT = OFF_SB + NSB * SB_BYTES;
  static constexpr int OFF_BAR = OFF_OUT + OUT_BYTES;
  static constexpr int SMEM = OFF_BAR + BAR_PAGE;
  static_assert(SMEM <= SMEM_LIMIT, "shared memory budget");
  // Tensor memory.  An M = 64 accumulator occupies lanes 0-15 of each 32-lane sub-partition, so two of them share
  // the same columns (second one at lane offset 16): both score tiles in 64 columns, both accumulators in NOUT
  // columns.  The state increment is double-buffered too: in lanes when R == 64, in columns when R == 128.
  static constexpr int NSC = 2;
  static constexpr int NACC = 2;
  static constexpr int TM_SC = 0, TM_ACC = 64, TM_DS = 64 + NOUT;
  static constexpr int DS_COLS = R == 128 ? 2 * CC : CC;
  // EMIT: a POP forward walk over full 64-token chunks that still delivers the state after every block: a block end
  // that falls inside a chunk (block sizes that are multiples of 16) gets its state from a PARTIAL increment, the
  // first p/16 k-steps of K^T Veta in a tile of its own:  S_block = gamma^p S + gamma^-(L-p) rs (K[:p]^T Veta[:p]).
  // Built where tensor memory has the room: the 64 x 64 tiles.
  static constexpr bool EMIT = MODE == MODE_FWD && R == 64 && CC == 64;
  static constexpr int TM_DSP = TM_DS + DS_COLS;
  static constexpr int TM_USED = TM_DSP + (EMIT ? CC : 0);
  static constexpr int TM_COLS = TM_USED <= 256 ? 256 : 512;
  static_assert(TM_USED <= 512, "tensor memory budget");
  static_assert(SOLO || TM_COLS == 256, "two CTAs per SM need at most 256 columns each");
  // state registers per state-warp thread; NHALF warps share one tensor-memory sub-partition
  static constexpr int NHALF = STATE_WARPS / 4;
  static constexpr int WCOLS = CC / NHALF;                   // state columns handled by one warp
  static constexpr int NS = R == 128 ? WCOLS : WCOLS / 2;
};

// SO ("state only"): the walk computes nothing but the state recurrence from a zero start and leaves its end value, fp32,
// in p.seg_states - the first pass of a T-segmented call.
// SF32: the call's state tensors (start / end state, block states and their gradients, suffix start states) are fp32.
template <int MODE, int REV, int R, int CC, bool SO, bool SF32, bool DEEP = false>
__global__ void __launch_bounds__(Cfg<MODE, R, CC, DEEP>::NTHREADS, Cfg<MODE, R, CC, DEEP>::MIN_CTAS)
scan_kernel(const __grid_constant__ ScanParams p) {
  using G = Cfg<MODE, R, CC, DEEP>;
  extern __shared__ __align__(1024) uint8_t sm[];
  const uint32_t sbase = smem_u32(sm);
  if (sbase & 1023) {                                  // the swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x7ff);
    return;
  }
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + G::OFF_BAR + OFF_ABORT);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + G::OFF_BAR + OFF_TMEM_SLOT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, h = blockIdx.y;
  // (a STATE_ONLY pass covers all pieces but the one the walk reaches last - the last one forward, the first one in
  // reverse - whose end value nobody needs ahead of time: the walk proper produces it)
  const int nz = SO ? p.n_seg - 1 : p.n_seg;
  const int b = p.n_seg > 1 ? (int)blockIdx.z / nz : (int)blockIdx.z;
  const int seg = p.n_seg > 1 ? (int)blockIdx.z % nz + ((SO && REV) ? 1 : 0) : 0;
  // this CTA walks tokens [t0, t_end) of the sequence; chunk positions are absolute (t0 is a chunk and block multiple)
  const int t0 = seg * p.seg_len;
  const int t_end = p.n_seg > 1 ? min(t0 + p.seg_len, p.T) : p.T;
  const bool by_cols = MODE == MODE_FWD || p.col_split != 0;
  const int row0 = by_cols ? 0 : tile * R;              // state rows [row0, row0+R) of dk
  const int col0 = by_cols ? tile * CC : 0;             // state cols [col0, col0+CC) of dv
  const float lg = p.log2g[h];
  const float rs = rsqrtf((float)p.dk);
  const int NC = chunk_count(t_end - t0, p.sched_bs);
  auto bar = [&](int slot) { return sbase + G::OFF_BAR + slot * 8; };
  constexpr int ARR_SCORE = N_SCORE, ARR_STATE = G::N_STATE;   // every thread of a role arrives (one elected lane per warp
                                                                // after a warp sync was measured: no faster)
  auto warp_arrive = [&](uint32_t b_) { mbar_arrive(b_); };
  auto stage_of = [&](int n) { return n % G::STAGES; };
  auto stage_ph = [&](int n) { return (uint32_t)((n / G::STAGES) & 1); };
  // tensor-memory address (lane offset in the upper half-word) of buffer n & 1 of each accumulator kind
  auto tm_sc = [&](int n) { return (uint32_t)(G::TM_SC + ((n & 1) ? (16u << 16) : 0u)); };
  auto tm_acc = [&](int n) { return (uint32_t)(G::TM_ACC + ((n & 1) ? (16u << 16) : 0u)); };
  auto tm_ds = [&](int n) { return R == 128 ? (uint32_t)(G::TM_DS + (n & 1) * CC) : (uint32_t)(G::TM_DS + ((n & 1) ? (16u << 16) : 0u)); };

  if (tid == 0) {
    for (int s = 0; s < G::STAGES; ++s) {
      mbar_init(bar(B_FULL + s), 1); mbar_init(bar(B_EMPTY + s), SO ? 1 : G::NMMA); mbar_init(bar(B_VRDY + s), ARR_STATE);
    }
    for (int j = 0; j < 2; ++j) {
      mbar_init(bar(B_SCFULL + j), 1); mbar_init(bar(B_PRDY + j), ARR_SCORE);
      mbar_init(bar(B_ACCFULL + j), 1); mbar_init(bar(B_ACCFREE + j), ARR_SCORE);
    }
    for (int j = 0; j < 2; ++j) { mbar_init(bar(B_DSFULL + j), 1); mbar_init(bar(B_DSFREE + j), ARR_STATE); }
    for (int j = 0; j < 2; ++j) { mbar_init(bar(B_SBRDY + j), ARR_STATE); mbar_init(bar(B_SBFREE + j), 1); }
    mbar_init(bar(B_DSPFULL), 1); mbar_init(bar(B_DSPFREE), ARR_STATE);
    fence_mbar_init();
    *abort_flag = 0;
    *reinterpret_cast<volatile long long*>(sm + G::OFF_BAR + OFF_LIMIT) = p.tune.wait_cycles;
    prefetch_tmap(&p.map_x); prefetch_tmap(&p.map_k); prefetch_tmap(&p.map_v); prefetch_tmap(&p.map_out);
  }
  if (warp == 1) { tmem_alloc(sbase + G::OFF_BAR + OFF_TMEM_SLOT, G::TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  // EMIT walks (forward, full chunks): tokens from the start of chunk n to the block end that falls strictly inside
  // it, or 0 when there is none (block sizes above 64 are the only ones walked this way: at most one per chunk)
  const bool emit = G::EMIT && !REV && p.sched_bs == 0 && p.block_size > 0 && p.block_states != nullptr;
  auto mid_end = [&](int n) {
    const int a = t0 + n * C, L = min(C, t_end - a);
    const int e = (a / p.block_size + 1) * p.block_size;
    return (e < a + L && e / p.block_size - 1 < p.n_blocks) ? e - a : 0;
  };
  Chunk first{REV ? t_end : t0, 0};
  advance<REV>(first, t_end, p.sched_bs);

  // =============================================================================================
  if (warp == 0) {                                   // ---------------- TMA producer
    if (lane == 0 && NC > 0) {
      Chunk ck = first;
      int issued = 0;
      for (int c = 0; c < NC; ++c) {
        const int s = stage_of(c);
        if (!mbar_wait(bar(B_EMPTY + s), stage_ph(c) ^ 1, abort_flag)) { FPB_GIVE_UP(0x100 | B_EMPTY); break; }
        FPB_TRACE(14, c);
        if (c == p.tune.withhold_chunk) { advance<REV>(ck, t_end, p.sched_bs); continue; }   // diagnostics: this chunk never arrives
        const uint32_t st = sbase + G::OFF_STAGE + s * G::STAGE_BYTES;
        mbar_arrive_expect_tx(bar(B_FULL + s), SO ? G::K_BYTES + G::V_BYTES : G::STAGE_BYTES);
        const int xcol0 = MODE == MODE_FWD ? row0 : col0;
        if (!SO) {
#pragma unroll
          for (int cb = 0; cb < G::W1 / 64; ++cb) tma_load_4d(st + cb * 8192, &p.map_x, bar(B_FULL + s), xcol0 + cb * 64, ck.a, h, b);
        }
#pragma unroll
        for (int cb = 0; cb < R / 64; ++cb) tma_load_4d(st + G::X_BYTES + cb * 8192, &p.map_k, bar(B_FULL + s), row0 + cb * 64, ck.a, h, b);
#pragma unroll
        for (int cb = 0; cb < CC / 64; ++cb) tma_load_4d(st + G::X_BYTES + G::K_BYTES + cb * 8192, &p.map_v, bar(B_FULL + s), col0 + cb * 64, ck.a, h, b);
        ++issued;
        advance<REV>(ck, t_end, p.sched_bs);
      }
      if (*abort_flag) {   // let the copies in flight land before the CTA's shared memory is released
        // (with a withheld chunk the stage numbering of the last copies is off by one: those were consumed anyway)
        for (int i = max(0, issued - G::STAGES); i < issued && p.tune.withhold_chunk < 0; ++i) {
          const long long w0 = clock64();
          while (!mbar_try_wait(bar(B_FULL + stage_of(i)), stage_ph(i)) && clock64() - w0 < wait_limit(abort_flag)) {}
        }
      }
    }
  } else if (warp == 1 || (G::NMMA >= 2 && warp == G::MMAB_WARP) || (G::NMMA == 3 && warp == G::MMAC_WARP)) {   // ---------------- MMA issuer(s)
    // The whole warp runs this loop with warp-uniform control flow and data (barrier tests are made uniform by a
    // vote), so that descriptors and counters stay in the uniform datapath; one elected lane issues.
    //
    // A chunk is four product groups - scores, increment, state term, intra-chunk term.  Two ways of issuing them:
    // one warp that polls for whichever product has its inputs (`issue_loop`: the small tiles, and every state-only
    // pass), or three warps with one blocking loop each (the 128-wide tiles, see Cfg::NMMA).  A stage goes back to the
    // producer when every issuing warp has committed its last product of the stage's chunk.
    if (NC > 0 && !(SO && warp != 1)) {
      const bool leader = elect_one();
      constexpr uint32_t ID_SC = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_STATE = MODE == MODE_FWD ? idesc_bf16(64, CC, 0, 1) : idesc_bf16(64, R, 0, 0);
      constexpr uint32_t ID_INTRA = idesc_bf16(64, G::NOUT, 0, 1);
      constexpr uint32_t ID_DS = idesc_bf16(R, CC, 1, 1);
      // Descriptors are built once; inside the issue loops an operand address advances by adding to the
      // 14-bit address field (16-byte units), so one tcgen05.mma costs this thread two additions.
      //   K-major tile [cb][64 rows][128 B]: k-step ks (16 elements) -> + (ks/4) * (column-block stride) + (ks%4) * 32 bytes
      //   MN-major tile: k-step ks (16 rows) -> + ks * 2048 bytes; lbo = column-block stride
      constexpr uint32_t STAGE16 = G::STAGE_BYTES >> 4;
      const uint64_t d_x = smem_desc(sbase + G::OFF_STAGE, 16, 1024);                                  // X, K-major
      const uint64_t d_kk = smem_desc(sbase + G::OFF_STAGE + G::X_BYTES, 16, 1024);                    // K, K-major
      const uint64_t d_km = smem_desc(sbase + G::OFF_STAGE + G::X_BYTES, 8192, 1024);                  // K, MN-major
      const uint64_t d_vk = smem_desc(sbase + G::OFF_STAGE + G::X_BYTES + G::K_BYTES, 16, 1024);       // V, K-major
      const uint64_t d_vm = smem_desc(sbase + G::OFF_STAGE + G::X_BYTES + G::K_BYTES, 8192, 1024);     // V, MN-major
      const uint64_t d_sb = MODE == MODE_FWD ? smem_desc(sbase + G::OFF_SB, R * 128, 1024)             // Sb: MN-major (FWD)
                                             : smem_desc(sbase + G::OFF_SB, 16, 1024);                 //     K-major (DQ)
      const uint64_t d_p = smem_desc(sbase + G::OFF_P, 16, 1024);                                       // P', K-major
      auto kstep = [](int ks, uint32_t cb_stride) { return (uint64_t)((ks >> 2) * (cb_stride >> 4) + (ks & 3) * 2); };
      auto mstep = [](int ks) { return (uint64_t)(ks * 128); };
      FPB_PROF_DECL();
      auto ready = [&](int slot, uint32_t parity) {
        FPB_PROF_BEGIN();
        const bool ok = __all_sync(0xffffffffu, mbar_test_wait(bar(slot), parity)) != 0;
        FPB_PROF_END(0);
        return ok;
      };
      // one polling warp for all four products (DO_A: scores, increment, POP partial increments; DO_B: state and
      // intra-chunk terms - both set wherever this loop is used)
      auto issue_loop = [&](auto do_a, auto do_b) {
        constexpr bool DO_A = decltype(do_a)::value, DO_B = decltype(do_b)::value;
        constexpr bool BOTH = DO_A && DO_B;
        // Next chunk to issue for each of the four products, and the next stage to hand back to the producer.
        // Each product of chunk n is issued when its inputs are there; the tensor pipe runs them in issue order.
        int n_sc = 0, n_ds = 0, n_qs = 0, n_pv = 0, n_rel = 0;
        int n_dsp = (emit && !SO) ? 0 : 0x7fffffff, m_dsp = 0;   // chunks whose partial increment is settled; partials issued
        // a stage goes back to the producer as soon as this warp's products of its chunk have been issued (issuing
        // blocks while the tensor pipe is busy, so this is checked after every group, not once per round)
        auto release = [&]() {
          while ((!DO_B || SO || n_rel < n_pv) && (!DO_A || ((SO || n_rel < n_sc) && n_rel < n_ds && n_rel < n_dsp))) {
            if (leader) { { FPB_PROF_BEGIN(); umma_commit(bar(B_EMPTY + stage_of(n_rel))); FPB_PROF_END(1); } FPB_TRACE(5, n_rel); }
            ++n_rel;
          }
        };
        // A barrier test costs this thread on the order of a hundred cycles while the tensor pipe is streaming
        // operands out of shared memory, so each barrier phase is tested until it has been seen complete once and
        // never again.  "V scaled" implies "tiles landed" (the state warps waited for them), so the products wait
        // for that one barrier only.
        int n_data = 0, n_full = 0, n_pdone = 0;
        auto data_ready = [&](int n) {
          if (n < n_data) return true;
          if (!ready(B_VRDY + stage_of(n_data), stage_ph(n_data))) return false;
          ++n_data;
          return n < n_data;
        };
        // The scores of a MODE_FWD walk read X and K only, not the tile the state warps rescale in place: they may go
        // as soon as the copies have landed, so that the chain scores -> P' -> intra-chunk term starts a rescaling early.
        auto scores_ready = [&](int n) {
          if (MODE != MODE_FWD || !p.tune.sc_early) return data_ready(n);
          if (n < n_data || n < n_full) return true;
          if (n_full < n_data) n_full = n_data;
          if (!ready(B_FULL + stage_of(n_full), stage_ph(n_full))) return false;
          ++n_full;
          return n < n_full;
        };
        // The score tile of chunk n may be overwritten once P' of chunk n - NSC has been taken out of it.  The warp that
        // also issues the intra-chunk terms knows that from its own counter (that term waited for P'); warp A alone
        // tests the P' barrier itself (NP == NSC in the split configurations, so the phase is unambiguous).
        auto score_tile_free = [&](int n) {
          if constexpr (BOTH) return n < n_pv + G::NSC;
          else {
            if (n < G::NSC || n - G::NSC < n_pdone) return true;
            if (!ready(B_PRDY + n_pdone % G::NP, (n_pdone / G::NP) & 1)) return false;
            ++n_pdone;
            return n - G::NSC < n_pdone;
          }
        };
        Patience patience{0, 0};
        while (n_rel < NC) {             // until every product of this warp for every chunk has been issued
          bool progress = false;
          // Order of the tests = priority: the products that feed the longest chains first (scores -> P' -> intra term;
          // increment -> state -> next chunk's state term).
          // scores Sc = X K^T (FWD) | X Veta^T (DQ)
          if (DO_A && !SO && n_sc < NC && score_tile_free(n_sc) && scores_ready(n_sc)) {
            const uint64_t so = (uint64_t)(stage_of(n_sc) * STAGE16);
            { FPB_PROF_BEGIN(); tc_fence_after(); FPB_PROF_END(3); }
            const uint32_t d = tm + tm_sc(n_sc);
            const uint64_t bk = (MODE == MODE_FWD ? d_kk : d_vk) + so;
            if (leader) {
              FPB_PROF_BEGIN();
FPB_UNROLL_MMA
              for (int ks = 0; ks < (FPB_ABL(32) ? 1 : G::W1 / 16); ++ks) umma_bf16(d, d_x + so + kstep(ks, 8192), bk + kstep(ks, 8192), ID_SC, ks > 0);
              FPB_PROF_END(2);
              { FPB_PROF_BEGIN(); umma_commit(bar(B_SCFULL + n_sc % G::NSC)); FPB_PROF_END(1); }
              FPB_TRACE(0, n_sc);
            }
            ++n_sc; progress = true;
          }
          // state increment dS = K^T Veta: depends on no other product and feeds the only chunk-to-chunk dependency
          if (DO_A && n_ds < NC && data_ready(n_ds) && (n_ds < 2 || ready(B_DSFREE + (n_ds & 1), ((n_ds >> 1) & 1) ^ 1))) {
            const uint64_t so = (uint64_t)(stage_of(n_ds) * STAGE16);
            { FPB_PROF_BEGIN(); tc_fence_after(); FPB_PROF_END(3); }
            if (leader) {
              FPB_PROF_BEGIN();
FPB_UNROLL_MMA
              for (int ks = 0; ks < (FPB_ABL(32) ? 1 : C / 16); ++ks) umma_bf16(tm + tm_ds(n_ds), d_km + so + mstep(ks), d_vm + so + mstep(ks), ID_DS, ks > 0);
              FPB_PROF_END(2);
              { FPB_PROF_BEGIN(); umma_commit(bar(B_DSFULL + (n_ds & 1))); FPB_PROF_END(1); }
              FPB_TRACE(4, n_ds);
            }
            ++n_ds; progress = true;
            release();
          }
          // EMIT: partial increment of the chunk whose full increment has just been issued (same operands, first k-steps)
          if (DO_A && G::EMIT && !SO && n_dsp < n_ds) {
            const int pmid = mid_end(n_dsp);
            if (pmid == 0) { ++n_dsp; progress = true; release(); }
            else if (m_dsp == 0 || ready(B_DSPFREE, (m_dsp - 1) & 1)) {
              const uint64_t so = (uint64_t)(stage_of(n_dsp) * STAGE16);
              { FPB_PROF_BEGIN(); tc_fence_after(); FPB_PROF_END(3); }
              if (leader) {
                FPB_PROF_BEGIN();
                for (int ks = 0; ks < pmid / 16; ++ks) umma_bf16(tm + G::TM_DSP, d_km + so + mstep(ks), d_vm + so + mstep(ks), ID_DS, ks > 0);
                FPB_PROF_END(2);
                { FPB_PROF_BEGIN(); umma_commit(bar(B_DSPFULL)); FPB_PROF_END(1); }
              }
              ++m_dsp; ++n_dsp; progress = true;
              release();
            }
          }
          // state term: ACC = X Sb (FWD) | X Sb^T (DQ)
          if (DO_B && !SO && n_qs < NC && data_ready(n_qs) && (n_qs < G::NACC || ready(B_ACCFREE + n_qs % G::NACC, ((n_qs / G::NACC) & 1) ^ 1)) &&
              ready(B_SBRDY + n_qs % G::NSB, (n_qs / G::NSB) & 1)) {
            const uint64_t so = (uint64_t)(stage_of(n_qs) * STAGE16);
            if (leader) FPB_TRACE(2, n_qs);
            { FPB_PROF_BEGIN(); tc_fence_after(); FPB_PROF_END(3); }
            const uint32_t acc = tm + tm_acc(n_qs);
            const uint64_t sbo = (uint64_t)((n_qs % G::NSB) * (G::SB_BYTES >> 4));      // which copy of the state
            if (leader) {
              if (MODE == MODE_FWD) {
                FPB_PROF_BEGIN();
FPB_UNROLL_MMA
                for (int ks = 0; ks < (FPB_ABL(32) ? 1 : R / 16); ++ks) umma_bf16(acc, d_x + so + kstep(ks, 8192), d_sb + sbo + mstep(ks), ID_STATE, ks > 0);
                FPB_PROF_END(2);
              } else {
                FPB_PROF_BEGIN();
FPB_UNROLL_MMA
                for (int ks = 0; ks < (FPB_ABL(32) ? 1 : CC / 16); ++ks) umma_bf16(acc, d_x + so + kstep(ks, 8192), d_sb + sbo + kstep(ks, R * 128), ID_STATE, ks > 0);
                FPB_PROF_END(2);
              }
              { FPB_PROF_BEGIN(); umma_commit(bar(B_SBFREE + n_qs % G::NSB)); FPB_PROF_END(1); }    // that copy may be overwritten once this has run
              FPB_TRACE(1, n_qs);
            }
            ++n_qs; progress = true;
          }
          // intra-chunk term: ACC += P' Veta (FWD) | P' K (DQ); needs the state term of the same chunk issued before
          if (DO_B && !SO && n_pv < n_qs && ready(B_PRDY + n_pv % G::NP, (n_pv / G::NP) & 1)) {   // the state term has seen the data
            const uint64_t so = (uint64_t)(stage_of(n_pv) * STAGE16);
            if (leader) FPB_TRACE(15, n_pv);
            { FPB_PROF_BEGIN(); tc_fence_after(); FPB_PROF_END(3); }
            const uint32_t acc = tm + tm_acc(n_pv);
            const uint64_t a = d_p + (uint64_t)((n_pv % G::NP) * (G::P_BYTES >> 4));
            const uint64_t bm = (MODE == MODE_FWD ? d_vm : d_km) + so;
            if (leader) {
              FPB_PROF_BEGIN();
FPB_UNROLL_MMA
              for (int ks = 0; ks < (FPB_ABL(32) ? 1 : C / 16); ++ks) umma_bf16(acc, a + kstep(ks, 0), bm + mstep(ks), ID_INTRA, 1);
              FPB_PROF_END(2);
              { FPB_PROF_BEGIN(); umma_commit(bar(B_ACCFULL + n_pv % G::NACC)); FPB_PROF_END(1); }
              FPB_TRACE(3, n_pv);
            }
            ++n_pv; progress = true;
            release();
          }
          release();
          if (progress) patience.progress();
          else if (__any_sync(0xffffffffu, patience.exhausted(abort_flag))) {
            if (leader) FPB_GIVE_UP((DO_A ? 0x200 : 0x500) | ((DO_A ? n_ds : n_pv) & 0xff));
            break;
          }
        }
      };
      // ---- three blocking issue loops (NMMA == 3), one warp each
      auto wait_or_quit = [&](int slot, uint32_t parity, int code) {
        if (mbar_wait(bar(slot), parity, abort_flag)) return true;
        if (leader) FPB_GIVE_UP(code);
        return false;
      };
      auto scores_loop = [&]() {                        // warp 1: Sc(n) = X K^T | X Veta^T
        const bool early = MODE == MODE_FWD && p.tune.sc_early;
        for (int n = 0; n < NC; ++n) {
          // the score tile of chunk n - NSC must have been read out (P' of that chunk written)
          if (n >= G::NSC && !wait_or_quit(B_PRDY + (n - G::NSC) % G::NP, ((n - G::NSC) / G::NP) & 1, 0x200 | (n & 0xff))) return;
          if (!wait_or_quit((early ? B_FULL : B_VRDY) + stage_of(n), stage_ph(n), 0x200 | (n & 0xff))) return;
          tc_fence_after();
          const uint64_t so = (uint64_t)(stage_of(n) * STAGE16);
          const uint32_t d = tm + tm_sc(n);
          const uint64_t bk = (MODE == MODE_FWD ? d_kk : d_vk) + so;
          if (leader) {
FPB_UNROLL_MMA
            for (int ks = 0; ks < G::W1 / 16; ++ks) umma_bf16(d, d_x + so + kstep(ks, 8192), bk + kstep(ks, 8192), ID_SC, ks > 0);
            umma_commit(bar(B_SCFULL + n % G::NSC));
            umma_commit(bar(B_EMPTY + stage_of(n)));
            FPB_TRACE(0, n);
          }
          __syncwarp();
        }
      };
      auto increment_loop = [&]() {                     // warp C: dS(n) = K^T Veta, and the POP partial increments
        int m_dsp = 0;
        for (int n = 0; n < NC; ++n) {
          if (!wait_or_quit(B_VRDY + stage_of(n), stage_ph(n), 0x600 | (n & 0xff))) return;
          if (n >= 2 && !wait_or_quit(B_DSFREE + (n & 1), ((n >> 1) & 1) ^ 1, 0x600 | (n & 0xff))) return;
          tc_fence_after();
          const uint64_t so = (uint64_t)(stage_of(n) * STAGE16);
          if (leader) {
FPB_UNROLL_MMA
            for (int ks = 0; ks < C / 16; ++ks) umma_bf16(tm + tm_ds(n), d_km + so + mstep(ks), d_vm + so + mstep(ks), ID_DS, ks > 0);
            umma_commit(bar(B_DSFULL + (n & 1)));
            FPB_TRACE(4, n);
          }
          if (G::EMIT && emit) {
            const int pmid = mid_end(n);
            if (pmid > 0) {
              if (m_dsp > 0 && !wait_or_quit(B_DSPFREE, (m_dsp - 1) & 1, 0x600 | (n & 0xff))) return;
              tc_fence_after();
              if (leader) {
                for (int ks = 0; ks < pmid / 16; ++ks) umma_bf16(tm + G::TM_DSP, d_km + so + mstep(ks), d_vm + so + mstep(ks), ID_DS, ks > 0);
                umma_commit(bar(B_DSPFULL));
              }
              ++m_dsp;
            }
          }
          if (leader) { umma_commit(bar(B_EMPTY + stage_of(n))); FPB_TRACE(5, n); }
          __syncwarp();
        }
      };
      auto accumulator_loop = [&]() {                   // warp B: ACC(n) = X Sb, then += P' Veta (same accumulator, in order)
        for (int n = 0; n < NC; ++n) {
          if (!wait_or_quit(B_VRDY + stage_of(n), stage_ph(n), 0x500 | (n & 0xff))) return;
          if (n >= G::NACC && !wait_or_quit(B_ACCFREE + n % G::NACC, ((n / G::NACC) & 1) ^ 1, 0x500 | (n & 0xff))) return;
          if (!wait_or_quit(B_SBRDY + n % G::NSB, (n / G::NSB) & 1, 0x500 | (n & 0xff))) return;
          tc_fence_after();
          const uint64_t so = (uint64_t)(stage_of(n) * STAGE16);
          const uint32_t acc = tm + tm_acc(n);
          const uint64_t sbo = (uint64_t)((n % G::NSB) * (G::SB_BYTES >> 4));
          if (leader) {
            FPB_TRACE(2, n);
            if (MODE == MODE_FWD) {
FPB_UNROLL_MMA
              for (int ks = 0; ks < R / 16; ++ks) umma_bf16(acc, d_x + so + kstep(ks, 8192), d_sb + sbo + mstep(ks), ID_STATE, ks > 0);
            } else {
FPB_UNROLL_MMA
              for (int ks = 0; ks < CC / 16; ++ks) umma_bf16(acc, d_x + so + kstep(ks, 8192), d_sb + sbo + kstep(ks, R * 128), ID_STATE, ks > 0);
            }
            umma_commit(bar(B_SBFREE + n % G::NSB));
            FPB_TRACE(1, n);
          }
          if (!wait_or_quit(B_PRDY + n % G::NP, (n / G::NP) & 1, 0x500 | (n & 0xff))) return;
          tc_fence_after();
          const uint64_t a = d_p + (uint64_t)((n % G::NP) * (G::P_BYTES >> 4));
          const uint64_t bm = (MODE == MODE_FWD ? d_vm : d_km) + so;
          if (leader) {
            FPB_TRACE(15, n);
FPB_UNROLL_MMA
            for (int ks = 0; ks < C / 16; ++ks) umma_bf16(acc, a + kstep(ks, 0), bm + mstep(ks), ID_INTRA, 1);
            umma_commit(bar(B_ACCFULL + n % G::NACC));
            umma_commit(bar(B_EMPTY + stage_of(n)));
            FPB_TRACE(3, n);
          }
          __syncwarp();
        }
      };
      if constexpr (G::NMMA == 3 && !SO) {
        static_assert(G::NP == G::NSC, "the scores warp reads the P' barrier as 'score tile free'");
        if (warp == 1) scores_loop();
        else if (warp == G::MMAB_WARP) accumulator_loop();
        else increment_loop();
      } else {
        issue_loop(std::true_type{}, std::true_type{});
      }
      if (warp == 1) FPB_PROF_STORE();
    }
  } else if (warp < STATE_WARP0) {                   // ---------------- score warps
    const int t = tid - SCORE_WARP0 * 32;            // 0..127
    const int q4 = warp & 3;                         // tensor-memory sub-partition of this warp
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int r_lo = q4 * 16 + (lane >> 2);          // this thread's two accumulator rows: r_lo, r_lo + 8
    const int cpair = (lane & 3) * 2;

    // P'(n): causal side of Sc times gamma^-L (and rs in forward walks), bf16, swizzled K-major tile
    auto make_p = [&](int n, int L) {
      tc_fence_after();
      if (FPB_ABL(4)) { tc_fence_before(); if (!FPB_ABL(64)) fence_async_smem(); warp_arrive(bar(B_PRDY + n % G::NP)); return; }
      uint32_t r[32];
      tmem_ld_16x256b_x8(tm + lane_base + tm_sc(n), r);
      tmem_wait_ld();
      tc_fence_before();
      const float cs = REV ? exp2f(-(float)L * lg) : exp2f(-(float)L * lg) * rs;
      uint8_t* pt = sm + G::OFF_P + (n % G::NP) * G::P_BYTES;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int col = g * 8 + cpair;
        auto keep = [&](int cc, int rr) { return REV ? cc >= rr : cc <= rr; };
        const float a0 = keep(col, r_lo) ? __uint_as_float(r[4 * g]) * cs : 0.f;
        const float a1 = keep(col + 1, r_lo) ? __uint_as_float(r[4 * g + 1]) * cs : 0.f;
        const float b0 = keep(col, r_lo + 8) ? __uint_as_float(r[4 * g + 2]) * cs : 0.f;
        const float b1 = keep(col + 1, r_lo + 8) ? __uint_as_float(r[4 * g + 3]) * cs : 0.f;
        *reinterpret_cast<uint32_t*>(pt + r_lo * 128 + ((g ^ (r_lo & 7)) << 4) + cpair * 2) = pack_bf16(a0, a1);
        *reinterpret_cast<uint32_t*>(pt + (r_lo + 8) * 128 + ((g ^ ((r_lo + 8) & 7)) << 4) + cpair * 2) = pack_bf16(b0, b1);
      }
      if (!FPB_ABL(64)) fence_async_smem();
      warp_arrive(bar(B_PRDY + n % G::NP));
      if (t == 0) FPB_TRACE(7, n);
    };

    // E(n): out_i = rowscale_i * ACC_i -> staging tile -> TMA store.  Each warp owns 16 rows of the accumulator (its
    // tensor-memory sub-partition) and stores them itself - its 2 KB slice of every 64-column block of the staging
    // tile is a whole number of 1024-byte swizzle patterns, so it is a valid TMA source on its own - which leaves
    // the four score warps free of one another: no warp waits at a barrier for the slowest.
    auto epilogue = [&](int n, Chunk ck) {
      // this warp's previous TMA stores must have finished reading its slice of the staging tile
      if (lane == 0) tma_store_wait_read0();
      __syncwarp();
      if (t == 0) FPB_TRACE(9, n);
      tc_fence_after();
      if (FPB_ABL(8)) { tc_fence_before(); warp_arrive(bar(B_ACCFREE + n % G::NACC)); return; }
      // row scale: zeta_i (forward walks) or eta_j * rs (reverse walks)
      const float z_lo = REV ? exp2f((float)(ck.L - 1 - r_lo) * lg) * rs : exp2f((float)(r_lo + 1) * lg);
      const float z_hi = REV ? exp2f((float)(ck.L - 9 - r_lo) * lg) * rs : exp2f((float)(r_lo + 9) * lg);
      uint8_t* stg = sm + G::OFF_OUT;
#pragma unroll
      for (int half = 0; half < G::NOUT / 64; ++half) {
        uint32_t r[32];
        tmem_ld_16x256b_x8(tm + lane_base + tm_acc(n) + half * 64, r);
        tmem_wait_ld();
        if (half == G::NOUT / 64 - 1) { tc_fence_before(); warp_arrive(bar(B_ACCFREE + n % G::NACC)); }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t lo = pack_bf16(__uint_as_float(r[4 * g]) * z_lo, __uint_as_float(r[4 * g + 1]) * z_lo);
          const uint32_t hi = pack_bf16(__uint_as_float(r[4 * g + 2]) * z_hi, __uint_as_float(r[4 * g + 3]) * z_hi);
          *reinterpret_cast<uint32_t*>(stg + half * 8192 + r_lo * 128 + ((g ^ (r_lo & 7)) << 4) + cpair * 2) = lo;
          *reinterpret_cast<uint32_t*>(stg + half * 8192 + (r_lo + 8) * 128 + ((g ^ ((r_lo + 8) & 7)) << 4) + cpair * 2) = hi;
        }
      }
      const bool whole_box = ck.L == C || ck.a + ck.L >= p.T;    // rows beyond L are past the sequence end: TMA clips them
      const int wrow0 = q4 * 16;                                // this warp's rows [wrow0, wrow0 + 16)
      const int ocol0 = MODE == MODE_FWD ? col0 : row0;
      if (whole_box) {
        if (!FPB_ABL(64)) fence_async_smem();
        __syncwarp();
        if (lane == 0 && ck.a + wrow0 < p.T) {
          if (MODE == MODE_DQ && p.col_split) {
#pragma unroll
            for (int cb = 0; cb < G::NOUT / 64; ++cb)
              tma_reduce_add_4d(&p.map_out, sbase + G::OFF_OUT + cb * 8192 + wrow0 * 128, ocol0 + cb * 64, ck.a + wrow0, h, b);
          } else {
#pragma unroll
            for (int cb = 0; cb < G::NOUT / 64; ++cb)
              tma_store_4d(&p.map_out, sbase + G::OFF_OUT + cb * 8192 + wrow0 * 128, ocol0 + cb * 64, ck.a + wrow0, h, b);
          }
          tma_store_commit();
        }
      } else {   // chunk cut short by a block end: rows >= L belong to another chunk, store rows < L only
        __syncwarp();
        bf16* go = p.out + (int64_t)b * p.out_sb + (int64_t)h * p.out_sh + ocol0;
        const int rows = min(16, ck.L - wrow0);
        for (int idx = lane; idx < rows * (G::NOUT / 8); idx += 32) {
          const int row = wrow0 + idx / (G::NOUT / 8), ch = idx % (G::NOUT / 8);
          const uint4 val = *reinterpret_cast<const uint4*>(stg + (ch >> 3) * 8192 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
          *reinterpret_cast<uint4*>(go + (int64_t)(ck.a + row) * p.out_st + ch * 8) = val;
        }
        __syncwarp();   // these generic reads of the slice come before its next rewrite
      }
      if (t == 0) FPB_TRACE(10, n);
    };

    // E(n) without the staging tile: with the 32-lane load shape thread t of a warp reads tensor-memory lane
    // 32*q4 + t, i.e. row 16*q4 + (t & 15) of accumulator buffer t >> 4 (the two buffers interleave in lanes), 32
    // consecutive columns at a time; the threads of buffer n & 1 scale, pack and store 64 bytes each per load.  No
    // thread waits for another, rows >= L are simply not stored, and the shared-memory port is left to the MMAs.
    auto epilogue_direct = [&](int n, Chunk ck) {
      tc_fence_after();
      if (FPB_ABL(8)) { tc_fence_before(); warp_arrive(bar(B_ACCFREE + n % G::NACC)); return; }
      const int row = q4 * 16 + (lane & 15);
      const bool mine = (lane >> 4) == (n & 1) && row < ck.L;
      const float z = REV ? exp2f((float)(ck.L - 1 - row) * lg) * rs : exp2f((float)(row + 1) * lg);
      const int ocol0 = MODE == MODE_FWD ? col0 : row0;
      bf16* go = p.out + (int64_t)b * p.out_sb + (int64_t)h * p.out_sh + (int64_t)(ck.a + row) * p.out_st + ocol0;
#pragma unroll 1
      for (int c0 = 0; c0 < G::NOUT; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(tm + lane_base + G::TM_ACC + c0, r);
        tmem_wait_ld();
        if (c0 + 32 == G::NOUT) { tc_fence_before(); warp_arrive(bar(B_ACCFREE + n % G::NACC)); }
        if (mine) {
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint4 val;
            val.x = pack_bf16(__uint_as_float(r[8 * v4]) * z, __uint_as_float(r[8 * v4 + 1]) * z);
            val.y = pack_bf16(__uint_as_float(r[8 * v4 + 2]) * z, __uint_as_float(r[8 * v4 + 3]) * z);
            val.z = pack_bf16(__uint_as_float(r[8 * v4 + 4]) * z, __uint_as_float(r[8 * v4 + 5]) * z);
            val.w = pack_bf16(__uint_as_float(r[8 * v4 + 6]) * z, __uint_as_float(r[8 * v4 + 7]) * z);
            *reinterpret_cast<uint4*>(go + c0 + 8 * v4) = val;
          }
        }
      }
      if (t == 0) FPB_TRACE(10, n);
    };

    if (NC > 0 && !SO) {
      // P' may run ahead of the epilogues by the number of P' buffers: buffer n % NP is free again once the
      // intra-chunk product of chunk n - NP has run, which epilogue n - NP has waited for
      int n_p = 0, n_e = 0, n_acc = 0;      // n_acc: chunks whose accumulator this thread has seen complete
      Chunk ck_p = first, ck_e = first;
      Patience patience{0, 0};
      while (n_e < NC) {
        // an accumulator's barrier phase stays put until its epilogue has released the buffer, so it can be
        // tested once, ahead of the epilogue, and P' of the next chunk made first: that is what the tensor pipe
        // is waiting for, the epilogue only drains
        if (n_acc < n_p && n_acc < n_e + G::NACC && mbar_test_wait(bar(B_ACCFULL + n_acc % G::NACC), (n_acc / G::NACC) & 1)) {
          if (t == 0) FPB_TRACE(8, n_acc);
          ++n_acc;
        }
        if (n_p < NC && n_p < n_acc + G::NP && mbar_test_wait(bar(B_SCFULL + n_p % G::NSC), (n_p / G::NSC) & 1)) {
          if (t == 0) FPB_TRACE(6, n_p);
          make_p(n_p, ck_p.L);
          ++n_p; advance<REV>(ck_p, t_end, p.sched_bs);
          patience.progress();
        } else if (n_e < n_acc) {
          if (G::DIRECT_OUT) epilogue_direct(n_e, ck_e);
          else epilogue(n_e, ck_e);
          ++n_e; advance<REV>(ck_e, t_end, p.sched_bs);
          patience.progress();
        } else if (patience.exhausted(abort_flag)) {
          FPB_GIVE_UP(0x300 | (n_e & 0xff));
          break;
        } else {
          // idle: sleep in hardware on the barrier most likely to complete next (leaves the issue slots to the
          // warps that have work, wakes at once when that barrier completes)
          const bool want_p = n_p < NC && n_p < n_acc + G::NP;
          if (want_p) mbar_try_wait_hint(bar(B_SCFULL + n_p % G::NSC), (n_p / G::NSC) & 1, p.tune.idle_ns);
          else mbar_try_wait_hint(bar(B_ACCFULL + n_acc % G::NACC), (n_acc / G::NACC) & 1, p.tune.idle_ns);
        }
      }
      if (!G::DIRECT_OUT && lane == 0) tma_store_wait_all0();
    }
  } else if (warp < STATE_WARP0 + G::STATE_WARPS) {  // ---------------- state warps
    const int t = tid - STATE_WARP0 * 32;            // 0..N_STATE-1
    const int q4 = warp & 3;
    const int half = (warp - STATE_WARP0) >> 2;      // which slice of the CC state columns
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int wcol0 = half * G::WCOLS;
    float S[G::NS];

    // element enumeration of this thread's registers: i -> (row, col) inside the (R, CC) tile
    //   R == 128: row = 32*q4 + lane, col = wcol0 + i
    //   R ==  64: row = 16*q4 + lane/4 + 8*((i>>1)&1), col = wcol0 + 8*(i>>2) + 2*(lane&3) + (i&1)
    auto row_of = [&](int i) { return R == 128 ? q4 * 32 + lane : q4 * 16 + (lane >> 2) + 8 * ((i >> 1) & 1); };
    auto col_of = [&](int i) { return R == 128 ? wcol0 + i : wcol0 + 8 * (i >> 2) + 2 * (lane & 3) + (i & 1); };

    const int64_t state_elems = (int64_t)p.dk * p.dv;
    // where the walk's start value comes from and where its end value goes.  Forward walks start from the
    // given state; reverse walks start from the gradient of the returned state and end in dS_0.  For a
    // suffix call, batch index = (row, m): suffix m of a row starts from s0[row] (m == 0) or from block
    // state m-1, its end state is dropped (zero gradient), and the reverse walk's end goes to the
    // gradient of that start state.
    // (the call's states are bf16 or fp32: SF32; the segment scratch is always fp32)
    const void* x_start = nullptr;
    void* x_end = nullptr;
    constexpr std::bool_constant<SF32> state_t{};
    constexpr std::true_type scratch_t{};
    constexpr int esz = SF32 ? 4 : 2;
    auto at = [&](const void* base, int64_t elems) { return (void*)((const char*)base + elems * esz); };
    // suffix calls: the batch index is (row, group of sfx_G consecutive suffixes)
    const int groups = p.sfx_M > 0 ? p.sfx_M / p.sfx_G : 1;
    const int sfx_row = b / groups, sfx_m0 = (b % groups) * p.sfx_G;
    auto sfx_start = [&](int m) -> const void* {       // where suffix m of this row starts from (forward walks)
      if (m == 0) return p.s0 ? at(p.s0, sfx_row * p.s0_sb + h * p.s0_sh) : nullptr;
      return p.sfx_blocks ? at(p.sfx_blocks, (((int64_t)sfx_row * p.sfx_N + (m - 1)) * p.H + h) * state_elems) : nullptr;
    };
    if (SO || p.n_seg > 1) {
      // T-segments: a STATE_ONLY pass leaves the local end value in this segment's scratch slot; the walk proper
      // starts from the value the scan put there, and the piece it reaches last ends in the call's end state
      float* slot = p.seg_states + (((int64_t)b * p.H + h) * p.n_seg + seg) * state_elems;
      if (SO) x_end = slot;
      else {
        x_start = slot;
        if (seg == (REV ? 0 : p.n_seg - 1) && p.s_out) x_end = at(p.s_out, b * p.so_sb + h * p.so_sh);
      }
    } else if (p.sfx_M > 0) {
      const int row = sfx_row, m = sfx_m0;
      void* blk = (m > 0 && p.sfx_blocks) ? at(p.sfx_blocks, (((int64_t)row * p.sfx_N + (m - 1)) * p.H + h) * state_elems) : nullptr;
      if (!REV) x_start = sfx_start(m);
      else x_end = m == 0 ? (p.s_out ? at(p.s_out, row * p.so_sb + h * p.so_sh) : nullptr) : blk;
    } else {
      if (p.s0) x_start = at(p.s0, b * p.s0_sb + h * p.s0_sh);
      if (p.s_out) x_end = at(p.s_out, b * p.so_sb + h * p.so_sh);
    }

    auto load_global = [&](const void* src_, auto f32, bool accumulate) {
      if constexpr (decltype(f32)::value) {
        const float* src = (const float*)src_;
        if (R == 128) {
          const float* rowp = src + (int64_t)(row0 + row_of(0)) * p.dv + col0 + wcol0;
#pragma unroll
          for (int i = 0; i < G::NS; i += 4) {
            const float4 val = *reinterpret_cast<const float4*>(rowp + i);
            S[i] = (accumulate ? S[i] : 0.f) + val.x; S[i + 1] = (accumulate ? S[i + 1] : 0.f) + val.y;
            S[i + 2] = (accumulate ? S[i + 2] : 0.f) + val.z; S[i + 3] = (accumulate ? S[i + 3] : 0.f) + val.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < G::NS; i += 2) {
            const float2 f = *reinterpret_cast<const float2*>(src + (int64_t)(row0 + row_of(i)) * p.dv + col0 + col_of(i));
            S[i] = (accumulate ? S[i] : 0.f) + f.x;
            S[i + 1] = (accumulate ? S[i + 1] : 0.f) + f.y;
          }
        }
      } else {
      const bf16* src = (const bf16*)src_;
      if (R == 128) {
        const bf16* rowp = src + (int64_t)(row0 + row_of(0)) * p.dv + col0 + wcol0;
#pragma unroll
        for (int i = 0; i < G::NS; i += 8) {
          const uint4 val = *reinterpret_cast<const uint4*>(rowp + i);
          const uint32_t* w = reinterpret_cast<const uint32_t*>(&val);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[e]));
            S[i + 2 * e] = (accumulate ? S[i + 2 * e] : 0.f) + f.x;
            S[i + 2 * e + 1] = (accumulate ? S[i + 2 * e + 1] : 0.f) + f.y;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < G::NS; i += 2) {
          const __nv_bfloat162 v2 = *reinterpret_cast<const __nv_bfloat162*>(src + (int64_t)(row0 + row_of(i)) * p.dv + col0 + col_of(i));
          const float2 f = __bfloat1622float2(v2);
          S[i] = (accumulate ? S[i] : 0.f) + f.x;
          S[i + 1] = (accumulate ? S[i + 1] : 0.f) + f.y;
        }
      }
      }
    };
    // reverse walks: add the gradient of block state n where block n ends (chunk end == (n+1) * block_size)
    auto inject = [&](int end) {
      if (REV && p.block_size > 0 && p.block_grads && end % p.block_size == 0 && end / p.block_size - 1 < p.n_blocks)
        load_global(at(p.block_grads, (((int64_t)b * p.n_blocks + (end / p.block_size - 1)) * p.H + h) * state_elems),
                    state_t, true);
    };
    auto store_global = [&](void* dst_, auto f32) {
      if constexpr (decltype(f32)::value) {
        float* dst = (float*)dst_;
        if (R == 128) {
          float* rowp = dst + (int64_t)(row0 + row_of(0)) * p.dv + col0 + wcol0;
#pragma unroll
          for (int i = 0; i < G::NS; i += 4) *reinterpret_cast<float4*>(rowp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < G::NS; i += 2)
            *reinterpret_cast<float2*>(dst + (int64_t)(row0 + row_of(i)) * p.dv + col0 + col_of(i)) = make_float2(S[i], S[i + 1]);
        }
      } else {
      bf16* dst = (bf16*)dst_;
      if (R == 128) {
        bf16* rowp = dst + (int64_t)(row0 + row_of(0)) * p.dv + col0 + wcol0;
#pragma unroll
        for (int i = 0; i < G::NS; i += 8) {
          uint4 val;
          val.x = pack_bf16(S[i], S[i + 1]); val.y = pack_bf16(S[i + 2], S[i + 3]);
          val.z = pack_bf16(S[i + 4], S[i + 5]); val.w = pack_bf16(S[i + 6], S[i + 7]);
          *reinterpret_cast<uint4*>(rowp + i) = val;
        }
      } else {
#pragma unroll
        for (int i = 0; i < G::NS; i += 2)
          *reinterpret_cast<uint32_t*>(dst + (int64_t)(row0 + row_of(i)) * p.dv + col0 + col_of(i)) = pack_bf16(S[i], S[i + 1]);
      }
      }
    };
    // bf16 copy of the state in shared memory: [CC/64 column blocks][R rows][128 bytes], 16-byte
    // pieces XOR-swizzled by (row & 7) — an MN-major B operand (FWD) or a K-major B operand (DQ).
    auto publish_sb = [&](int n) {
      uint8_t* sb = sm + G::OFF_SB + (n % G::NSB) * G::SB_BYTES;
      if (FPB_ABL(2)) { if (!FPB_ABL(64)) fence_async_smem(); warp_arrive(bar(B_SBRDY + n % G::NSB)); return; }
      if (R == 128) {
        const int row = row_of(0);
#pragma unroll
        for (int i = 0; i < G::NS; i += 8) {
          const int col = col_of(i);
          uint4 val;
          val.x = pack_bf16(S[i], S[i + 1]); val.y = pack_bf16(S[i + 2], S[i + 3]);
          val.z = pack_bf16(S[i + 4], S[i + 5]); val.w = pack_bf16(S[i + 6], S[i + 7]);
          *reinterpret_cast<uint4*>(sb + (col >> 6) * (R * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4)) = val;
        }
      } else {
#pragma unroll
        for (int i = 0; i < G::NS; i += 2) {
          const int row = row_of(i), col = col_of(i);
          *reinterpret_cast<uint32_t*>(sb + (col >> 6) * (R * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + (col & 7) * 2) =
              pack_bf16(S[i], S[i + 1]);
        }
      }
      if (!FPB_ABL(64)) fence_async_smem();
      warp_arrive(bar(B_SBRDY + n % G::NSB));
    };
    // in-place row scale of the V tile of chunk n: eta_j = gamma^(L-1-j) (forward walks) or
    // zeta_i = gamma^(i+1) (reverse walks, the tile holds dO); rows >= L are zeroed
    auto scale_v = [&](int n, int L) {
      const int s = stage_of(n);
      uint8_t* vt = sm + G::OFF_STAGE + s * G::STAGE_BYTES + G::X_BYTES + G::K_BYTES;
      for (int idx = t; idx < (FPB_ABL(1) ? 0 : C * CC / 8); idx += G::N_STATE) {
        const int row = (idx >> 3) & 63;
        uint4* ptr = reinterpret_cast<uint4*>(vt + idx * 16);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (row < L) {
          const float e = exp2f((float)(REV ? row + 1 : L - 1 - row) * lg);
          val = *ptr;
          uint32_t* w = reinterpret_cast<uint32_t*>(&val);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[i]));
            w[i] = pack_bf16(f.x * e, f.y * e);
          }
        }
        *ptr = val;
      }
      if (!FPB_ABL(64)) fence_async_smem();
      warp_arrive(bar(B_VRDY + s));
    };

    if (x_start) {
      if (!SO && p.n_seg > 1) load_global(x_start, scratch_t, false);
      else load_global(x_start, state_t, false);
    }
    else {
#pragma unroll
      for (int i = 0; i < G::NS; ++i) S[i] = 0.f;
    }
    const float ds_scale = REV ? 1.0f : rs;   // forward: S += rs K^T Veta;  reverse: G += Q^T (zeta.dO)
    if (NC > 0) {
      // three tasks, each in chunk order, run as their inputs arrive:
      //   V(n)  scale the V tile of chunk n                         (needs the tiles of chunk n)
      //   U(n)  S <- gamma^L S + dS(n)                              (needs the increment of chunk n)
      //   Sb(n) publish the bf16 copy of the state at the start of chunk n; it must happen between U(n-1) and U(n),
      //         and after the state-term product of chunk n-1 has finished reading the previous copy
      int n_v = 0, n_u = 0, m_part = 0;
      bool publish_due = !SO, partial_due = emit && !SO && mid_end(0) > 0;   // partial_due: chunk n_u has a block end inside
      Chunk ck_v = first, ck_u = first;
      inject(first.a + first.L);
      constexpr int TSTEP = 16;                            // state registers per tensor-memory load
      static_assert(G::NS % TSTEP == 0, "a state-warp thread holds whole loads of its slice");
      // block state from the partial increment of chunk n_u (its barrier has completed)
      auto emit_block_state = [&]() {
        tc_fence_after();
        const int pmid = mid_end(n_u);
        const float gp = exp2f((float)pmid * lg), up = exp2f(-(float)(ck_u.L - pmid) * lg) * rs;
        void* dst_ = at(p.block_states, (((int64_t)b * p.n_blocks + ((ck_u.a + pmid) / p.block_size - 1)) * p.H + h) * state_elems);
#pragma unroll
        for (int i0 = 0; i0 < G::NS; i0 += TSTEP) {
          uint32_t r[TSTEP];
          tmem_ld_16x256b_x4(tm + lane_base + G::TM_DSP + wcol0 + i0 * 2, r);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < TSTEP; i += 2) {
            const float lo = fmaf(gp, S[i0 + i], up * __uint_as_float(r[i])), hi = fmaf(gp, S[i0 + i + 1], up * __uint_as_float(r[i + 1]));
            const int64_t off = (int64_t)(row0 + row_of(i0 + i)) * p.dv + col0 + col_of(i0 + i);
            if (SF32) *reinterpret_cast<float2*>((float*)dst_ + off) = make_float2(lo, hi);
            else *reinterpret_cast<uint32_t*>((bf16*)dst_ + off) = pack_bf16(lo, hi);
          }
        }
        tc_fence_before();
        warp_arrive(bar(B_DSPFREE));
        ++m_part; partial_due = false;
      };
      // U(n_u): S <- gamma^L S + dS(n_u) (its barrier has completed), and what follows a chunk's end
      // with_emit (EMIT walks): the partial increment of the chunk is complete as well - the block state and the update
      // are made in one pass over the registers, both tensor-memory loads in flight together
      auto update_state = [&](bool with_emit) {
        if (t == 0) FPB_TRACE(12, n_u);
        tc_fence_after();
        const float gl = exp2f((float)ck_u.L * lg);
        auto plain_update = [&]() {
          // 16 registers at a time keeps the state warps inside the register budget
#pragma unroll
          for (int i0 = 0; i0 < (FPB_ABL(16) ? 0 : G::NS); i0 += TSTEP) {
            uint32_t r[TSTEP];
            if constexpr (R == 128) tmem_ld_32x32b_x16(tm + lane_base + tm_ds(n_u) + wcol0 + i0, r);
            else tmem_ld_16x256b_x4(tm + lane_base + tm_ds(n_u) + wcol0 + i0 * 2, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < TSTEP; ++i) S[i0 + i] = fmaf(gl, S[i0 + i], ds_scale * __uint_as_float(r[i]));
          }
          tc_fence_before();
        };
        if constexpr (G::EMIT && DEEP) {     // (the deep variant has the registers for both tiles in flight)
          if (with_emit) {
            const int pmid = mid_end(n_u);
            const float gp = exp2f((float)pmid * lg), up = exp2f(-(float)(ck_u.L - pmid) * lg) * rs;
            void* dst_ = at(p.block_states, (((int64_t)b * p.n_blocks + ((ck_u.a + pmid) / p.block_size - 1)) * p.H + h) * state_elems);
#pragma unroll
            for (int i0 = 0; i0 < G::NS; i0 += TSTEP) {
              uint32_t rp[TSTEP], r[TSTEP];
              tmem_ld_16x256b_x4(tm + lane_base + G::TM_DSP + wcol0 + i0 * 2, rp);
              tmem_ld_16x256b_x4(tm + lane_base + tm_ds(n_u) + wcol0 + i0 * 2, r);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < TSTEP; i += 2) {
                const float lo = fmaf(gp, S[i0 + i], up * __uint_as_float(rp[i])), hi = fmaf(gp, S[i0 + i + 1], up * __uint_as_float(rp[i + 1]));
                const int64_t off = (int64_t)(row0 + row_of(i0 + i)) * p.dv + col0 + col_of(i0 + i);
                if (SF32) *reinterpret_cast<float2*>((float*)dst_ + off) = make_float2(lo, hi);
                else *reinterpret_cast<uint32_t*>((bf16*)dst_ + off) = pack_bf16(lo, hi);
                S[i0 + i] = fmaf(gl, S[i0 + i], ds_scale * __uint_as_float(r[i]));
                S[i0 + i + 1] = fmaf(gl, S[i0 + i + 1], ds_scale * __uint_as_float(r[i + 1]));
              }
            }
            tc_fence_before();
            warp_arrive(bar(B_DSPFREE));
            ++m_part; partial_due = false;
          } else plain_update();
        } else plain_update();
        warp_arrive(bar(B_DSFREE + (n_u & 1)));   // the increment has been read: the one after next may overwrite it
        const int end = ck_u.a + ck_u.L;
        if (!REV && !SO && p.block_size > 0 && p.block_states && end % p.block_size == 0 && end / p.block_size - 1 < p.n_blocks)
          store_global(at(p.block_states, (((int64_t)b * p.n_blocks + (end / p.block_size - 1)) * p.H + h) * state_elems), state_t);
        ++n_u;
        if (n_u < NC) {
          advance<REV>(ck_u, t_end, p.sched_bs);
          if (!REV && !SO && p.sfx_G > 1 && ck_u.a % p.block_size == 0) {
            // grouped suffixes: the next chunk opens the next suffix, which starts from its own state
            const void* src = sfx_start(sfx_m0 + ck_u.a / p.block_size);
            if (src) load_global(src, state_t, false);
            else {
#pragma unroll
              for (int i = 0; i < G::NS; ++i) S[i] = 0.f;
            }
          }
          inject(ck_u.a + ck_u.L);
          publish_due = !SO;
          partial_due = emit && !SO && mid_end(n_u) > 0;
        }
      };
      Patience patience{0, 0};
      while (n_u < NC) {
        bool progress = false;
        auto try_scale = [&]() {
          if (n_v < NC && mbar_test_wait(bar(B_FULL + stage_of(n_v)), stage_ph(n_v))) {
            scale_v(n_v, ck_v.L);
            if (t == 0) FPB_TRACE(11, n_v);
            ++n_v; advance<REV>(ck_v, t_end, p.sched_bs);
            progress = true;
          }
        };
        // 128-wide walks: the state copy and the state update come first - they sit on the chunk-to-chunk chain (copy ->
        // state term -> copy of the next chunk), the tile rescaling only has to stay ahead of the products (2 %).  The
        // small tiles, whose products are short, want the rescaling first (the other order cost the 64 x 64 dQ walk 30 %).
        if constexpr (!G::ONE) try_scale();
        if (publish_due) {
          // copy n_u goes into buffer n_u % NSB, which the state term of chunk n_u - NSB was the last to read
          if (n_u < G::NSB || mbar_test_wait(bar(B_SBFREE + n_u % G::NSB), (n_u / G::NSB - 1) & 1)) {
            publish_sb(n_u);
            if (t == 0) FPB_TRACE(13, n_u);
            publish_due = false; progress = true;
          }
        } else if (G::EMIT && partial_due) {
          if (mbar_test_wait(bar(B_DSPFULL), m_part & 1)) {
            // (the partial increment is issued right after the full one, so the latter is normally complete too)
            if (DEEP && mbar_test_wait(bar(B_DSFULL + (n_u & 1)), (n_u >> 1) & 1)) update_state(true);
            else emit_block_state();
            progress = true;
          }
        } else if (mbar_test_wait(bar(B_DSFULL + (n_u & 1)), (n_u >> 1) & 1)) {
          update_state(false);
          progress = true;
        }
        if constexpr (G::ONE) try_scale();
        if (progress) patience.progress();
        else if (patience.exhausted(abort_flag)) { FPB_GIVE_UP(0x400 | (n_u & 0xff)); break; }
        else if (publish_due) mbar_try_wait_hint(bar(B_SBFREE + n_u % G::NSB), (n_u / G::NSB - 1) & 1, p.tune.idle_ns);   // idle: sleep on the likely next
        else if (G::EMIT && partial_due) mbar_try_wait_hint(bar(B_DSPFULL), m_part & 1, p.tune.idle_ns);
        else mbar_try_wait_hint(bar(B_DSFULL + (n_u & 1)), (n_u >> 1) & 1, p.tune.idle_ns);
      }
    }
    if (x_end && !*abort_flag) {
      if (SO) store_global(x_end, scratch_t);
      else store_global(x_end, state_t);
    }
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tm, G::TM_COLS); }
}

template <int MODE, int REV, int R, int CC, bool SO, bool SF32, bool DEEP = false>
int launch_scan_t(const ScanParams& p, dim3 grid, cudaStream_t stream) {
  using G = Cfg<MODE, R, CC, DEEP>;
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(scan_kernel<MODE, REV, R, CC, SO, SF32, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM) != cudaSuccess)
      return FPB_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  scan_kernel<MODE, REV, R, CC, SO, SF32, DEEP><<<grid, G::NTHREADS, G::SMEM, stream>>>(p);
  return FPB_OK;
}
int sm_count_cached() {
  static std::atomic<int> cache[64];
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if ((n = cache[dev].load(std::memory_order_acquire)) == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev].store(n, std::memory_order_release);
  }
  return n;
}

#ifdef FPB_DIAGNOSTICS
int g_deep = 1;                  // 1: small tiles take the deep-pipeline variant when the grid has at most one CTA per SM
#else
constexpr int g_deep = 1;
#endif

template <int MODE, int R, int CC>
int launch_scan(const ScanParams& p, bool rev, bool state_only, dim3 grid, cudaStream_t stream) {
  const bool f32 = p.state_f32 != 0;
  if constexpr (MODE == MODE_FWD) {   // the state-only pass exists for the tilings of the output walks
    // (a state-only pass starts from zero and ends in fp32 scratch; only the block gradients of a reverse POP walk are typed)
    if (state_only) {
      if (!rev) return launch_scan_t<MODE, 0, R, CC, true, false>(p, grid, stream);
      return f32 ? launch_scan_t<MODE, 1, R, CC, true, true>(p, grid, stream) : launch_scan_t<MODE, 1, R, CC, true, false>(p, grid, stream);
    }
  }
  if (state_only) return FPB_ERR_BAD_SHAPE;
  if constexpr (R == 64 && CC == 64) {   // at most one CTA per SM: the deep-pipeline variant (forward walks, bf16 states)
    if (!f32 && !rev && g_deep && (long long)grid.x * grid.y * grid.z <= sm_count_cached())
      return launch_scan_t<MODE, 0, R, CC, false, false, true>(p, grid, stream);
  }
  if (f32) return rev ? launch_scan_t<MODE, 1, R, CC, false, true>(p, grid, stream) : launch_scan_t<MODE, 0, R, CC, false, true>(p, grid, stream);
  return rev ? launch_scan_t<MODE, 1, R, CC, false, false>(p, grid, stream) : launch_scan_t<MODE, 0, R, CC, false, false>(p, grid, stream);
}

// Scheduling choices.  A release build fixes them; the diagnostics build (-DFPB_DIAGNOSTICS) exports setters so that
// tests can run the alternative schedules against each other.
#ifdef FPB_DIAGNOSTICS
#define FPB_KNOB int
#else
#define FPB_KNOB constexpr int
#endif
FPB_KNOB g_tile_pref = 1;            // 1: 128x128 state tiles where they apply; 0: 64-wide tiles (two CTAs per SM)
FPB_KNOB g_sfx_group = 16;           // most suffixes one CTA walks back to back (1: one CTA per suffix)
FPB_KNOB g_sfx_min_ctas = 3 * 296;   // ... as long as that many CTAs remain (three waves of two CTAs per SM)
FPB_KNOB g_pop_emit = 1;             // 1: POP forward walks over full chunks where block states can come from partial increments
FPB_KNOB g_fused_bwd = 1;            // 1: dK, dV, dS_0 in one fused reverse walk where it applies; 0: two separate walks
FPB_KNOB g_segments = 1;             // 1: under-filled launches are cut into T-segments when the caller gave scratch memory
FPB_KNOB g_col_split = 1;            // 1: dv = 256 gradient walks cut dv into 128 x 128 tiles and add their partial results
#ifdef FPB_DIAGNOSTICS
long long* g_trace = nullptr;        // set by fpb_debug_trace
WalkTuning g_tuning{kWaitCycles, 200, 1, -1, 0};
#else
constexpr long long* g_trace = nullptr;
constexpr WalkTuning g_tuning{kWaitCycles, 200, 1, -1, 0};
#endif

bool aligned_state(const StateView& s, bool f32) {
  const int64_t m = f32 ? 4 : 8;
  return !s.data || ((uintptr_t)s.data % 16 == 0 && s.sb % m == 0 && s.sh % m == 0);
}

// Which (mode, dk, dv) combinations the kernel is instantiated for.
bool scan_supported(int mode, int dk, int dv) {
  (void)mode;
  return (dk == 64 || dk == 128) && (dv == 64 || dv == 128 || dv == 256);
}

struct PassArgs {
  int mode; bool rev;
  SeqView x, k, v, out;
  StateView start, end;          // start value of the walk (read) and where its end value goes (written)
  void* block_states; const void* block_grads;
  SuffixStates sfx;
  const float* gamma;
  int B, T, H, dk, dv, block_size, n_blocks;
  bool state_f32;
  float* scratch; int64_t scratch_bytes;   // fp32 scratch for T-segments, or null
};

bool pass_applicable(const PassArgs& a) {
  if (!scan_supported(a.mode, a.dk, a.dv)) return false;
  if (!tma_addressable(a.x, 2) || !tma_addressable(a.k, 2) || !tma_addressable(a.v, 2) || !tma_addressable(a.out, 2)) return false;
  if (!aligned_state(a.start, a.state_f32) || !aligned_state(a.end, a.state_f32)) return false;
  if ((uintptr_t)a.block_states % 16 || (uintptr_t)a.block_grads % 16 || (uintptr_t)a.sfx.blocks % 16) return false;
  return a.B <= 65535 && a.H <= 65535 && a.T > 0;
}

// state tile and CTAs per SM of the instance a pass runs on
struct Tiling { int R, CC, tiles, ctas_per_sm; bool col_split; };
// split_ok: a MODE_DQ walk may cut dv instead of dk.  Its output tile is then a partial sum over the CTA's dv columns,
// which TMA adds to the (zeroed) output in L2 - two addends per element when dv = 256, so the result does not depend on
// their order.  For dv = 256 that replaces the 64 x 256 tiles (M = 64 products over 256 columns, 5400 cycles per chunk)
// by the 128 x 128 instance.  Only walks whose chunks are all stored as whole tiles qualify (no POP blocks, no suffixes).
Tiling tiling_of(int mode, int dk, int dv, bool split_ok) {
  if (mode == MODE_FWD) {         // state tile: all dk rows x CC columns of dv
    if (dk == 128 && dv % 128 == 0 && g_tile_pref) return {128, 128, dv / 128, 1, false};
    if (dk == 128) return {128, 64, dv / 64, 2, false};
    return {64, 64, dv / 64, 2, false};
  }                               // state tile: R rows of dk x all dv columns
  if (dv == 128 && dk % 128 == 0 && g_tile_pref) return {128, 128, dk / 128, 1, false};
  if (dv == 64) return {64, 64, dk / 64, 2, false};
  if (dv == 128) return {64, 128, dk / 64, 2, false};
  if (dk == 128 && split_ok && g_col_split && g_tile_pref) return {128, 128, dv / 128, 1, true};
  return {64, 256, dk / 64, 1, false};
}
bool col_split_ok(int mode, int block_size, const SuffixStates& sfx) { return mode == MODE_DQ && block_size == 0 && sfx.M == 0; }

// Zeros over the (B, T, H, d) elements of a strided bf16 view, d a multiple of 8: a CTA takes ZERO_TOKENS tokens of a
// batch row and writes their H * d / 8 16-byte pieces each (32-bit index arithmetic: a 64-bit division per piece made
// the fill issue-bound at half the HBM write rate).
constexpr int ZERO_TOKENS = 16;
__global__ void __launch_bounds__(256) zero_seq_kernel(bf16* base, int64_t sb, int64_t st, int64_t sh, int T, int H, int d8) {
  const int t0 = blockIdx.x * ZERO_TOKENS, nt = min(ZERO_TOKENS, T - t0);
  bf16* row = base + (int64_t)blockIdx.y * sb + (int64_t)t0 * st;
  const uint32_t per_token = (uint32_t)(H * d8), total = (uint32_t)nt * per_token;
  for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
    const uint32_t t = i / per_token, r = i - t * per_token;
    const uint32_t h = r / (uint32_t)d8, c = r - h * (uint32_t)d8;
    *reinterpret_cast<uint4*>(row + (int64_t)t * st + (int64_t)h * sh + c * 8) = make_uint4(0u, 0u, 0u, 0u);
  }
}

int gcd_int(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }

// One launch of the kernel: the walk itself, or (state_only) the local end values of its T-segments.
int launch_one(const PassArgs& a, Segments sg, bool state_only, cudaStream_t stream) {
  const int mode = state_only ? MODE_FWD : a.mode;
  const int xw = mode == MODE_FWD ? a.dk : a.dv, ow = mode == MODE_FWD ? a.dv : a.dk;
  const int B = a.B, T = a.T, H = a.H, dk = a.dk, dv = a.dv;
  ScanParams p;
  int r;
  // Suffix calls are thousands of sequences of a few chunks.  Where the suffixes of a row follow one another in
  // memory, G of them are walked by one CTA as one sequence of G * T tokens whose state is replaced at every suffix
  // start (block size = suffix length, so no chunk straddles two suffixes): the CTA's set-up and pipeline fill are
  // paid once per G suffixes.  G is the largest divisor of M that still leaves a few waves of CTAs.
  int G = 1;
  SeqView x = state_only ? a.k : a.x, k = a.k, v = a.v, out = state_only ? a.v : a.out;   // a state-only pass reads k and v only
  int Bk = B, Tk = T, block_size = a.block_size;
  if (a.sfx.M > 1 && !a.rev && g_sfx_group && a.block_size == 0 && x.sb == (int64_t)T * x.st && k.sb == (int64_t)T * k.st &&
      v.sb == (int64_t)T * v.st && out.sb == (int64_t)T * out.st) {
    G = choose_suffix_group(a.sfx.M, (long long)(B / a.sfx.M) * H * (mode == MODE_FWD ? (dv + 127) / 128 : (dk + 127) / 128));
    if (G > 1) {
      Bk = B / G; Tk = T * G; block_size = T;
      x.sb *= G; k.sb *= G; v.sb *= G; out.sb *= G;
    }
  }
  if ((r = make_seq_map(&p.map_x, x, Bk, Tk, H, xw, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_k, k, Bk, Tk, H, dk, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_v, v, Bk, Tk, H, dv, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_out, out, Bk, Tk, H, ow, 16)) != FPB_OK) return r;   // one score warp's 16 rows
  p.out = (bf16*)out.data; p.out_sb = out.sb; p.out_st = out.st; p.out_sh = out.sh;
  const bool split = sg.n > 1;
  // a segmented walk starts from the scratch slots; its last piece writes the end value
  p.s0 = split ? nullptr : a.start.data; p.s0_sb = a.start.sb; p.s0_sh = a.start.sh;
  p.s_out = state_only ? nullptr : a.end.data; p.so_sb = a.end.sb; p.so_sh = a.end.sh;
  p.block_states = state_only ? nullptr : a.block_states;
  p.block_grads = a.block_grads;
  p.sfx_blocks = a.sfx.blocks; p.sfx_M = a.sfx.M; p.sfx_N = a.sfx.N; p.sfx_G = G;
  p.T = Tk; p.H = H; p.dk = dk; p.dv = dv; p.block_size = block_size; p.n_blocks = a.n_blocks;
  p.state_f32 = a.state_f32 ? 1 : 0;
  p.n_seg = sg.n; p.seg_len = sg.seg_len; p.seg_states = a.scratch;
  p.tune = g_tuning;
  // POP forward at 64 x 64: full chunks, block states from partial increments (block sizes above 64 that are multiples
  // of 16 but not of 64 - for those the block-aligned schedule already is the full-chunk one)
  const bool emit = g_pop_emit && mode == MODE_FWD && !a.rev && a.block_states && dk == 64 && dv == 64 &&
                    block_size > 64 && block_size % 16 == 0 && block_size % 64 != 0 && G == 1;
  p.sched_bs = emit ? 0 : block_size;
  p.status = device_status_ptr();
  p.trace = g_trace;
  if (!p.status) return FPB_ERR_LAUNCH;
  for (int h = 0; h < H; ++h) p.log2g[h] = (float)std::log2((double)a.gamma[h]);

  const Tiling t = tiling_of(mode, dk, dv, col_split_ok(mode, a.block_size, a.sfx));
  p.col_split = t.col_split ? 1 : 0;
  const dim3 grid(t.tiles, H, Bk * (state_only ? sg.n - 1 : sg.n));
#define FPB_SCAN_CASE(MODE_, R_, CC_) \
  if (mode == MODE_ && t.R == R_ && t.CC == CC_) return launch_scan<MODE_, R_, CC_>(p, a.rev, state_only, grid, stream)
  FPB_SCAN_CASE(MODE_FWD, 128, 128); FPB_SCAN_CASE(MODE_FWD, 128, 64); FPB_SCAN_CASE(MODE_FWD, 64, 64);
  FPB_SCAN_CASE(MODE_DQ, 128, 128); FPB_SCAN_CASE(MODE_DQ, 64, 64); FPB_SCAN_CASE(MODE_DQ, 64, 128); FPB_SCAN_CASE(MODE_DQ, 64, 256);
#undef FPB_SCAN_CASE
  return FPB_ERR_BAD_SHAPE;
}

// A pass = one launch, or three when the launch would leave most of the GPU idle and the caller gave scratch memory:
// local end values of T-segments, the scan over them, the walk proper from the segments' start values.
int launch_pass(const PassArgs& a, cudaStream_t stream, int* n_launched) {
  Segments sg{1, 0};
  if (g_segments && a.scratch && a.sfx.M == 0 && a.B * 16 <= 65535) {
    const Tiling t = tiling_of(a.mode, a.dk, a.dv, col_split_ok(a.mode, a.block_size, a.sfx));
    const int align = a.block_size > 0 ? C / gcd_int(C, a.block_size) * a.block_size : C;   // segment starts: chunk and block multiples
    sg = choose_segments((long long)t.tiles * a.H * a.B, t.ctas_per_sm, a.T, align, (long long)a.B * a.H, (long long)a.dk * a.dv,
                         a.scratch_bytes, a.B);
  }
  int r;
  if (sg.n > 1) {
    if ((r = launch_one(a, sg, true, stream)) != FPB_OK) return r;
    if ((r = launch_segment_combine(a.scratch, sg, a.B, a.T, a.H, a.dk, a.dv, a.gamma, a.rev, a.start, a.state_f32, stream)) != FPB_OK)
      return r;
    *n_launched += 2;
  }
  if (tiling_of(a.mode, a.dk, a.dv, col_split_ok(a.mode, a.block_size, a.sfx)).col_split) {
    launch_zero_seq(a.out, a.B, a.T, a.H, a.mode == MODE_FWD ? a.dv : a.dk, stream);   // the tiles' partial results are added to it
    ++*n_launched;
  }
  if ((r = launch_one(a, sg, false, stream)) != FPB_OK) return r;
  ++*n_launched;
  return FPB_OK;
}

}  // namespace

long long* debug_trace_ptr() { return g_trace; }
const WalkTuning& walk_tuning() { return g_tuning; }
bool segments_enabled() { return g_segments != 0; }
bool col_split_enabled() { return g_col_split != 0 && g_tile_pref != 0; }
void launch_zero_seq(const SeqView& v, int B, int T, int H, int d, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return;
  zero_seq_kernel<<<dim3((T + ZERO_TOKENS - 1) / ZERO_TOKENS, B), 256, 0, stream>>>((bf16*)v.data, v.sb, v.st, v.sh, T, H, d / 8);
}


int choose_suffix_group(int M, long long units) {
  for (int cand = g_sfx_group; cand > 1; --cand)
    if (M % cand == 0 && units * (M / cand) >= g_sfx_min_ctas) return cand;
  return 1;
}

#ifdef FPB_DIAGNOSTICS
// Hooks of the diagnostics build (not part of the public header).
// Install a device buffer of 64*16 int64 that the next launches fill with clock64() stamps of their first CTA; null removes it.
extern "C" void fpb_debug_trace(void* device_buffer) { g_trace = (long long*)device_buffer; }
// Choose between the 128x128 state tiles (1, default) and the 64-wide ones (0).
extern "C" void fpb_debug_tile_pref(int wide) { g_tile_pref = wide; }
// Upper limit of the suffixes one CTA walks back to back (1 = one CTA per suffix) and the number of CTAs that must remain.
extern "C" void fpb_debug_suffix_group(int g, int min_ctas) { g_sfx_group = g < 1 ? 1 : g; if (min_ctas > 0) g_sfx_min_ctas = min_ctas; }
// 0 makes every POP forward walk cut its chunks at block ends.
extern "C" void fpb_debug_pop_emit(int on) { g_pop_emit = on; }
// 0 runs the dV and dK walks as two launches instead of the fused reverse kernel.
extern "C" void fpb_debug_fused_bwd(int on) { g_fused_bwd = on; }
// 0 never cuts sequences into T-segments.
extern "C" void fpb_debug_segments(int on) { g_segments = on; }
// 0 keeps the dk-tiled 64 x 256 instances (and the two separate reverse walks) for dv = 256.
extern "C" void fpb_debug_col_split(int on) { g_col_split = on; }
// 0 keeps the two-CTAs-per-SM configuration of the small tiles for every grid size.
extern "C" void fpb_debug_deep(int on) { g_deep = on; }
// Wait limit in clock ticks (<= 0: the default of about a second), idle suspend hint in ns, early scores on / off, and the
// chunk the producers withhold (-1: none; makes every role's wait on it run out).
extern "C" void fpb_debug_ablate(int mask) { g_tuning.ablate = mask; }
extern "C" void fpb_debug_tuning(long long wait_cycles, int idle_ns, int sc_early, int withhold_chunk) {
  g_tuning.wait_cycles = wait_cycles > 0 ? wait_cycles : kWaitCycles;
  g_tuning.idle_ns = idle_ns > 0 ? idle_ns : 200;
  g_tuning.sc_early = sc_early;
  g_tuning.withhold_chunk = withhold_chunk;
}
#endif

int launch_umma_fwd(const UmmaFwdArgs& a, cudaStream_t stream, int* n_launched) {
  *n_launched = 0;
  if (a.dtype != FPB_BF16) return FPB_UMMA_NOT_APPLICABLE;
  PassArgs f{MODE_FWD, false, a.q, a.k, a.v, a.o, a.s0, a.s_out, a.block_states, nullptr, a.sfx, a.gamma,
             a.B, a.T, a.H, a.dk, a.dv, a.block_size, a.n_blocks, a.state_f32, a.scratch, a.scratch_bytes};
  if (!pass_applicable(f)) return FPB_UMMA_NOT_APPLICABLE;
  return launch_pass(f, stream, n_launched);
}

// Local end values of the T-segments of a walk over (k, v): used by the fused reverse kernel, whose own file has no
// state-only instance (its first pass is the reverse MODE_FWD walk with (k, v) := (q, dO)).
int launch_segment_states(SeqView k, SeqView v, bool rev, const void* block_grads, const float* gamma, int B, int T, int H, int dk,
                          int dv, int block_size, int n_blocks, bool state_f32, Segments sg, float* scratch, cudaStream_t stream) {
  const StateView none{nullptr, 0, 0};
  PassArgs a{MODE_FWD, rev, k, k, v, v, none, none, nullptr, block_grads, SuffixStates{0, 0, nullptr}, gamma,
             B, T, H, dk, dv, block_size, n_blocks, state_f32, scratch, 0};
  return launch_one(a, sg, true, stream);
}

// Backward = three independent walks: dQ (forward walk over the states), dV + dS_0 and dK (reverse
// walks over the state gradient).
int launch_umma_bwd(const UmmaBwdArgs& a, cudaStream_t stream, int* n_launched) {
  *n_launched = 0;
  if (a.dtype != FPB_BF16) return FPB_UMMA_NOT_APPLICABLE;
  const StateView none{nullptr, 0, 0};
  // dQ needs the states at chunk starts only, never a block state: its walk ignores the POP block structure and
  // takes full 64-token chunks (fewer chunks than the block-aligned schedule whenever the block is not a multiple of 64)
  PassArgs dq{MODE_DQ, false, a.dO, a.k, a.v, a.dQ, a.s0, none, nullptr, nullptr, a.sfx_in, a.gamma,
              a.B, a.T, a.H, a.dk, a.dv, 0, 0, a.state_f32, a.scratch, a.scratch_bytes};
  PassArgs dv{MODE_FWD, true, a.k, a.q, a.dO, a.dV, a.d_s_out, a.d_s0, nullptr, a.d_block_states, a.sfx_grad, a.gamma,
              a.B, a.T, a.H, a.dk, a.dv, a.block_size, a.n_blocks, a.state_f32, a.scratch, a.scratch_bytes};
  SuffixStates no_write = a.sfx_grad;
  no_write.blocks = nullptr;
  PassArgs dk{MODE_DQ, true, a.v, a.q, a.dO, a.dK, a.d_s_out, none, nullptr, a.d_block_states, no_write, a.gamma,
              a.B, a.T, a.H, a.dk, a.dv, a.block_size, a.n_blocks, a.state_f32, a.scratch, a.scratch_bytes};
  if ((!a.skip_dq && !pass_applicable(dq)) || (!a.skip_dkdv && (!pass_applicable(dv) || !pass_applicable(dk))))
    return FPB_UMMA_NOT_APPLICABLE;
  int r;
  if (!a.skip_dq && (r = launch_pass(dq, stream, n_launched)) != FPB_OK) return r;
  if (a.skip_dkdv) return FPB_OK;
  if (g_fused_bwd) {
    r = launch_bwd_fused(a, stream, n_launched);
    if (r == FPB_OK) return FPB_OK;
    if (r != FPB_UMMA_NOT_APPLICABLE) return r;
  }
  if ((r = launch_pass(dv, stream, n_launched)) != FPB_OK) return r;
  return launch_pass(dk, stream, n_launched);
}

}  // namespace fpb
