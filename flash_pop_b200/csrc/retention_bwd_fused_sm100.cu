// tcgen05 kernel for the REVERSE walk of the retention backward on sm_100a: dK, dV and dS_0 in one pass
// (replaces fused_retention_bwd_dk_dv_ds / pop_retention_bwd_dk_dv_ds of the reference,
// flash_pop/fused_retention/fused_chunk_bwd.py:218-346, flash_pop/pop_retention/pop_bwd.py:9-165).
//
// One CTA walks one (batch, head) sequence from its last chunk to its first, carrying
// G = d(loss)/d(state after the chunk) as fp32 in the registers of the state warps.  Per chunk of L <= 64
// tokens (gamma = head decay, rs = 1/sqrt(dk), zeta_i = gamma^(i+1), eta_j = gamma^(L-1-j)):
//   dOz   = zeta . dO                       in place in shared memory (rows >= L zeroed)
//   Sc1   = K Q^T          Sc2 = V dOz^T    64x64 fp32 score tiles in tensor memory
//   P1    = triu(Sc1) gamma^-L              P2 = triu(Sc2) gamma^-L        bf16, swizzled shared memory
//   ACCV  = K Gb + P1 dOz                   ACCK = V Gb^T + P2 Q           Gb = bf16 copy of G
//   dV_j  = eta_j rs ACCV_j                 dK_j = eta_j rs ACCK_j         epilogue, TMA stores
//   dG    = Q^T dOz ;   G <- gamma^L G + dG  (+ the POP block-state gradient where a block ends)
// which is the reference's  dV = A^T dO + (K.eta) dS,  dK = [P^T Q + (V.eta) dS^T] / sqrt(dk),
// dS <- gamma^L dS + Q^T (zeta.dO)  (fused_chunk_bwd.py:180-215) with the decay mask factored into row,
// column and constant scales exactly as in retention_scan_sm100.cu.  Compared with running the dV and the dK
// walk separately it reads Q, K, V, dO once (4 tensors instead of 6), scales dO once and carries one G.
//
// Roles and scheduling are those of retention_scan_sm100.cu: TMA producer, warp-uniform MMA issuer with an
// elected lane, four score warps (P1, P2, both epilogues), state warps (dO scaling, G update, Gb); every role
// polls its barriers and runs whichever task is ready; every wait is bounded.  Tensor memory (512 columns at
// dk = dv = 128): the M = 64 tiles are lane-interleaved (two per column range) — Sc1 x2, Sc2 x2, ACCV | ACCK —
// and dG is double-buffered.
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

constexpr int SCORE_WARP0 = 2, STATE_WARP0 = 6;
constexpr int N_SCORE = 128;

struct BwdParams {
  CUtensorMap map_q, map_k, map_v, map_do, map_dk, map_dv;
  CUtensorMap map_bg;                            // POP, 64 x 64, bf16 states: the block-state gradients, one 64 x 64 box per (row, block, head)
  bf16* dk_out; int64_t dk_sb, dk_st, dk_sh;
  bf16* dv_out; int64_t dv_sb, dv_st, dv_sh;
  // states are bf16 or fp32 (state_f32), strides in elements
  const void* g_start; int64_t gs_sb, gs_sh;     // gradient of the returned state (start of the reverse walk), or null
  void* g_end; int64_t ge_sb, ge_sh;             // dS_0 (end of the reverse walk), or null
  const void* block_grads;                       // POP: gradients of the block states (B, NB, H, dk, dv), or null
  void* sfx_blocks; int32_t sfx_M, sfx_N;        // suffix calls: gradients of the start states taken from block states
  int32_t sfx_G;                                 // suffixes one CTA walks back to back as one sequence (>= 1)
  int32_t T, H, dk, dv, block_size, n_blocks;
  int32_t state_f32;
  int32_t n_seg, seg_len;                        // T-segments (segment_scan.cu): blockIdx.z = batch * n_seg + segment
  const float* seg_states;                       // fp32 (B, H, n_seg, dk, dv): G after the last token of each segment
  WalkTuning tune;
  int32_t* status;
  long long* trace;
  float log2g[FPB_MAX_HEADS];
};

constexpr int MAXS = 5;          // most stages a configuration may have
enum { B_FULL = 0, B_EMPTY = MAXS, B_VRDY = 2 * MAXS, B_SCFULL = 3 * MAXS, B_PRDY = B_SCFULL + 2, B_ACCFULL = B_PRDY + 2,
       B_ACCFREE = B_ACCFULL + 1, B_DSFULL = B_ACCFREE + 1, B_DSFREE = B_DSFULL + 2, B_SBRDY = B_DSFREE + 2, B_SBFREE = B_SBRDY + 1,
       B_PFFULL = B_SBFREE + 1, B_PFFREE = B_PFFULL + 1, B_COUNT = B_PFFREE + 1 };
constexpr int OFF_TMEM_SLOT = B_COUNT * 8, OFF_ABORT = OFF_TMEM_SLOT + 4, OFF_LIMIT = OFF_ABORT + 4, BAR_PAGE = 256;
static_assert(OFF_LIMIT % 8 == 0 && OFF_LIMIT + 8 <= BAR_PAGE, "the wait limit sits right after the abort flag");

template <int DK, int DV>
struct BCfg {
  static constexpr int DMAX = DK > DV ? DK : DV;
  static constexpr int STATE_WARPS = DK * DV >= 128 * 128 ? 8 : 4;   // (eight at 64 x 64 measured 2.5 % slower)
  static constexpr int N_STATE = 32 * STATE_WARPS;
  // the 128 x 128 instance issues its seven product groups from two warps (see the MMA issuer); the second is the last warp
  static constexpr bool SPLIT = DK * DV >= 128 * 128;
  static constexpr int MMAB_WARP = STATE_WARP0 + STATE_WARPS;
  static constexpr int NTHREADS = STATE_WARP0 * 32 + N_STATE + (SPLIT ? 32 : 0);
  static constexpr int Q_BYTES = C * DK * 2, V_BYTES = C * DV * 2;           // Q and K tiles; V and dO tiles
  static constexpr int STAGE_BYTES = 2 * Q_BYTES + 2 * V_BYTES;
  static constexpr int OFF_Q = 0, OFF_K = Q_BYTES, OFF_V = 2 * Q_BYTES, OFF_DO = 2 * Q_BYTES + V_BYTES;   // inside a stage
  static constexpr int P_BYTES = C * C * 2;
  static constexpr int NP = 2;
  static constexpr int GB_BYTES = DK * DV * 2;
  // POP: the block-state gradient that the walk adds next, fetched one block ahead by a bulk copy (64 x 64, bf16 states)
  static constexpr int PF_BYTES = (DK == 64 && DV == 64) ? DK * DV * 2 : 0;
  static constexpr int FIXED = 2 * NP * P_BYTES + GB_BYTES + C * DV * 2 + C * DK * 2 + BAR_PAGE + PF_BYTES;
  static constexpr int SMEM_LIMIT = 226 * 1024;
  // as many stages as the shared memory of the SM holds (the CTA has it to itself): 3 at d = 128, 5 at d = 64, where a
  // chunk's few kilobytes leave the walk bound by the number of chunks in flight
  static constexpr int FIT = (SMEM_LIMIT - FIXED) / STAGE_BYTES;
  static constexpr int STAGES = FIT < MAXS ? FIT : MAXS;
  static_assert(STAGES >= 2, "at least two stages");
  static constexpr int OFF_STAGE = 0;
  static constexpr int OFF_P1 = STAGES * STAGE_BYTES;
  static constexpr int OFF_P2 = OFF_P1 + NP * P_BYTES;
  static constexpr int OFF_GB = OFF_P2 + NP * P_BYTES;
  static constexpr int OFF_OUTV = OFF_GB + GB_BYTES;
  static constexpr int OFF_OUTK = OFF_OUTV + C * DV * 2;
  static constexpr int OFF_PF = OFF_OUTK + C * DK * 2;       // (a swizzled TMA tile: 1024-byte aligned like the others)
  static constexpr int OFF_BAR = OFF_PF + PF_BYTES;
  static constexpr int SMEM = OFF_BAR + BAR_PAGE;
  static_assert(SMEM <= SMEM_LIMIT, "shared memory budget");
  // tensor memory: Sc1 (2 buffers in lanes) | Sc2 (2 buffers in lanes) | ACCV (lanes 0-15) + ACCK (lanes 16-31) | dG x2
  static constexpr int TM_SC1 = 0, TM_SC2 = 64, TM_ACC = 128, TM_DG = 128 + DMAX;
  static constexpr int DG_COLS = DK == 128 ? 2 * DV : DV;
  static constexpr int TM_USED = TM_DG + DG_COLS;
  static constexpr int TM_COLS = TM_USED <= 256 ? 256 : 512;
  static_assert(TM_USED <= 512, "tensor memory budget");
  static constexpr int NHALF = STATE_WARPS / 4;
  static constexpr int WCOLS = DV / NHALF;
  static constexpr int NS = DK == 128 ? WCOLS : WCOLS / 2;
};

// SF32: the call's state tensors (gradient of the returned state, dS_0, block-state gradients) are fp32.
template <int DK, int DV, bool SF32>
__global__ void __launch_bounds__(BCfg<DK, DV>::NTHREADS, 1) bwd_fused_kernel(const __grid_constant__ BwdParams p) {
  using G = BCfg<DK, DV>;
  extern __shared__ __align__(1024) uint8_t sm[];
  const uint32_t sbase = smem_u32(sm);
  if (sbase & 1023) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, 0x7fe);
    return;
  }
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + G::OFF_BAR + OFF_ABORT);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(sm + G::OFF_BAR + OFF_TMEM_SLOT);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  // dv = 2 DV: blockIdx.x is the half of dv this CTA takes.  dV and the G columns of the half are complete; dK is a
  // partial sum over the half's columns, which TMA adds to the (zeroed) output.
  const int vcol = (int)blockIdx.x * DV;
  const bool dv_split = gridDim.x > 1;
  const int b = p.n_seg > 1 ? (int)blockIdx.z / p.n_seg : (int)blockIdx.z;
  const int seg = p.n_seg > 1 ? (int)blockIdx.z % p.n_seg : 0;
  // this CTA walks tokens [t0, t_end) of the sequence; chunk positions are absolute (t0 is a chunk and block multiple)
  const int t0 = seg * p.seg_len;
  const int t_end = p.n_seg > 1 ? min(t0 + p.seg_len, p.T) : p.T;
  const float lg = p.log2g[h];
  const float rs = rsqrtf((float)p.dk);
  const int NC = chunk_count(t_end - t0, p.block_size);
  auto bar = [&](int slot) { return sbase + G::OFF_BAR + slot * 8; };
  auto stage_of = [&](int n) { return n % G::STAGES; };
  auto stage_ph = [&](int n) { return (uint32_t)((n / G::STAGES) & 1); };
  // tensor-memory addresses (lane offset in the upper half-word)
  auto lanes16 = [](int odd) { return odd ? (16u << 16) : 0u; };
  auto tm_sc1 = [&](int n) { return (uint32_t)G::TM_SC1 + lanes16(n & 1); };
  auto tm_sc2 = [&](int n) { return (uint32_t)G::TM_SC2 + lanes16(n & 1); };
  const uint32_t tm_accv = G::TM_ACC, tm_acck = G::TM_ACC + (16u << 16);
  auto tm_dg = [&](int n) { return DK == 128 ? (uint32_t)(G::TM_DG + (n & 1) * DV) : (uint32_t)G::TM_DG + lanes16(n & 1); };

  if (tid == 0) {
    for (int s = 0; s < G::STAGES; ++s) { mbar_init(bar(B_FULL + s), 1); mbar_init(bar(B_EMPTY + s), G::SPLIT ? 2 : 1); mbar_init(bar(B_VRDY + s), G::N_STATE); }
    for (int j = 0; j < 2; ++j) {
      mbar_init(bar(B_SCFULL + j), 1); mbar_init(bar(B_PRDY + j), N_SCORE);
      mbar_init(bar(B_DSFULL + j), 1); mbar_init(bar(B_DSFREE + j), G::N_STATE);
    }
    mbar_init(bar(B_ACCFULL), 1); mbar_init(bar(B_ACCFREE), N_SCORE);
    mbar_init(bar(B_SBRDY), G::N_STATE); mbar_init(bar(B_SBFREE), 1);
    mbar_init(bar(B_PFFULL), 1); mbar_init(bar(B_PFFREE), G::N_STATE);
    fence_mbar_init();
    *abort_flag = 0;
    *reinterpret_cast<volatile long long*>(sm + G::OFF_BAR + OFF_LIMIT) = p.tune.wait_cycles;
    prefetch_tmap(&p.map_q); prefetch_tmap(&p.map_k); prefetch_tmap(&p.map_v); prefetch_tmap(&p.map_do);
    prefetch_tmap(&p.map_dk); prefetch_tmap(&p.map_dv);
    if (G::PF_BYTES > 0 && !SF32 && p.block_grads) prefetch_tmap(&p.map_bg);
  }
  if (warp == 1) { tmem_alloc(sbase + G::OFF_BAR + OFF_TMEM_SLOT, G::TM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  Chunk first{t_end, 0};
  prev_chunk(first, p.block_size);

  // =============================================================================================
  if (warp == 0) {                                   // ---------------- TMA producer
    if (lane == 0 && NC > 0) {
      Chunk ck = first;
      int issued = 0;
      for (int c = 0; c < NC; ++c) {
        const int s = stage_of(c);
        if (!mbar_wait(bar(B_EMPTY + s), stage_ph(c) ^ 1, abort_flag)) { FPB_GIVE_UP(0x100 | B_EMPTY); break; }
        FPB_TRACE(14, c);
        if (c == p.tune.withhold_chunk) { prev_chunk(ck, p.block_size); continue; }   // diagnostics: this chunk never arrives
        const uint32_t st = sbase + G::OFF_STAGE + s * G::STAGE_BYTES;
        mbar_arrive_expect_tx(bar(B_FULL + s), G::STAGE_BYTES);
#pragma unroll
        for (int cb = 0; cb < DV / 64; ++cb) {      // dO first: it has to be scaled before anything can use it
          tma_load_4d(st + G::OFF_DO + cb * 8192, &p.map_do, bar(B_FULL + s), vcol + cb * 64, ck.a, h, b);
          tma_load_4d(st + G::OFF_V + cb * 8192, &p.map_v, bar(B_FULL + s), vcol + cb * 64, ck.a, h, b);
        }
#pragma unroll
        for (int cb = 0; cb < DK / 64; ++cb) {
          tma_load_4d(st + G::OFF_Q + cb * 8192, &p.map_q, bar(B_FULL + s), cb * 64, ck.a, h, b);
          tma_load_4d(st + G::OFF_K + cb * 8192, &p.map_k, bar(B_FULL + s), cb * 64, ck.a, h, b);
        }
        ++issued;
        prev_chunk(ck, p.block_size);
      }
      if (*abort_flag) {   // let the copies in flight land before the CTA's shared memory is released
        for (int i = max(0, issued - G::STAGES); i < issued && p.tune.withhold_chunk < 0; ++i) {
          const long long w0 = clock64();
          while (!mbar_try_wait(bar(B_FULL + stage_of(i)), stage_ph(i)) && clock64() - w0 < wait_limit(abort_flag)) {}
        }
      }
    }
  } else if (warp == 1 || (G::SPLIT && warp == G::MMAB_WARP)) {   // ---------------- MMA issuer(s) (warp-uniform, one elected lane)
    // The issuing thread is the walk's pacemaker (seven product groups, each with its barrier tests, descriptor
    // arithmetic and commit), so the 128 x 128 instance splits them over two warps along the line that needs no ordering
    // between them: warp A issues what depends on the tiles alone (both score products, the increment), warp B the
    // accumulator products (state terms, then intra-chunk terms).  A stage is released when both have committed.
    if (NC > 0) {
      const bool leader = elect_one();
      constexpr uint32_t ID_SC = idesc_bf16(64, 64, 0, 0);
      constexpr uint32_t ID_KG = idesc_bf16(64, DV, 0, 1);      // K Gb      : B = Gb, MN-major
      constexpr uint32_t ID_VG = idesc_bf16(64, DK, 0, 0);      // V Gb^T    : B = Gb, K-major
      constexpr uint32_t ID_P1 = idesc_bf16(64, DV, 0, 1);      // P1 dOz    : B = dOz, MN-major
      constexpr uint32_t ID_P2 = idesc_bf16(64, DK, 0, 1);      // P2 Q      : B = Q, MN-major
      constexpr uint32_t ID_DG = idesc_bf16(DK, DV, 1, 1);      // Q^T dOz
      constexpr uint32_t STAGE16 = G::STAGE_BYTES >> 4;
      const uint32_t st0 = sbase + G::OFF_STAGE;
      const uint64_t d_qk = smem_desc(st0 + G::OFF_Q, 16, 1024), d_qm = smem_desc(st0 + G::OFF_Q, 8192, 1024);
      const uint64_t d_kk = smem_desc(st0 + G::OFF_K, 16, 1024);
      const uint64_t d_vk = smem_desc(st0 + G::OFF_V, 16, 1024);
      const uint64_t d_ok = smem_desc(st0 + G::OFF_DO, 16, 1024), d_om = smem_desc(st0 + G::OFF_DO, 8192, 1024);
      const uint64_t d_gm = smem_desc(sbase + G::OFF_GB, DK * 128, 1024), d_gk = smem_desc(sbase + G::OFF_GB, 16, 1024);
      const uint64_t d_p1 = smem_desc(sbase + G::OFF_P1, 16, 1024), d_p2 = smem_desc(sbase + G::OFF_P2, 16, 1024);
      auto kstep = [](int ks, uint32_t cb_stride) { return (uint64_t)((ks >> 2) * (cb_stride >> 4) + (ks & 3) * 2); };
      auto mstep = [](int ks) { return (uint64_t)(ks * 128); };
      auto ready = [&](int slot, uint32_t parity) { return __all_sync(0xffffffffu, mbar_test_wait(bar(slot), parity)) != 0; };
      auto issue_loop = [&](auto do_a, auto do_b) {
      constexpr bool DO_A = decltype(do_a)::value, DO_B = decltype(do_b)::value;
      int n_sc = 0, n_ds = 0, n_qs = 0, n_pv = 0, n_rel = 0, n_data = 0, n_pdone = 0;
      auto data_ready = [&](int n) {     // "dO scaled" implies "tiles landed"; each phase is tested until seen once
        if (n < n_data) return true;
        if (!ready(B_VRDY + stage_of(n_data), stage_ph(n_data))) return false;
        ++n_data;
        return n < n_data;
      };
      // score buffers n & 1 are free once P1/P2 of chunk n - 2 were taken out: the warp that issues the intra terms knows it
      // from its own counter; warp A alone tests the P' barrier (two P' buffers, so the phase is unambiguous)
      auto score_tiles_free = [&](int n) {
        if constexpr (DO_A && DO_B) return n < n_pv + 2;
        else {
          if (n < 2 || n - 2 < n_pdone) return true;
          if (!ready(B_PRDY + (n_pdone & 1), (n_pdone >> 1) & 1)) return false;
          ++n_pdone;
          return n - 2 < n_pdone;
        }
      };
      auto release = [&]() {
        while ((!DO_B || n_rel < n_pv) && (!DO_A || (n_rel < n_ds && n_rel < n_sc))) {
          if (leader) { umma_commit(bar(B_EMPTY + stage_of(n_rel))); FPB_TRACE(5, n_rel); }
          ++n_rel;
        }
      };
      Patience patience{0, 0};
      while (n_rel < NC) {
        bool progress = false;
        // scores of chunk n into buffers n & 1; free once P1/P2 of chunk n-2 were taken out (seen by its intra terms)
        if (DO_A && n_sc < NC && score_tiles_free(n_sc) && data_ready(n_sc)) {
          const uint64_t so = (uint64_t)(stage_of(n_sc) * STAGE16);
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) umma_bf16(tm + tm_sc1(n_sc), d_kk + so + kstep(ks, 8192), d_qk + so + kstep(ks, 8192), ID_SC, ks > 0);
#pragma unroll
            for (int ks = 0; ks < DV / 16; ++ks) umma_bf16(tm + tm_sc2(n_sc), d_vk + so + kstep(ks, 8192), d_ok + so + kstep(ks, 8192), ID_SC, ks > 0);
            umma_commit(bar(B_SCFULL + (n_sc & 1)));
            FPB_TRACE(0, n_sc);
          }
          ++n_sc; progress = true;
        }
        // increment dG = Q^T dOz into buffer n & 1
        if (DO_A && n_ds < NC && data_ready(n_ds) && (n_ds < 2 || ready(B_DSFREE + (n_ds & 1), ((n_ds >> 1) & 1) ^ 1))) {
          const uint64_t so = (uint64_t)(stage_of(n_ds) * STAGE16);
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < C / 16; ++ks) umma_bf16(tm + tm_dg(n_ds), d_qm + so + mstep(ks), d_om + so + mstep(ks), ID_DG, ks > 0);
            umma_commit(bar(B_DSFULL + (n_ds & 1)));
            FPB_TRACE(4, n_ds);
          }
          ++n_ds; progress = true;
          release();
        }
        // state terms ACCV = K Gb, ACCK = V Gb^T (one accumulator pair: wait until the previous epilogue has read it)
        if (DO_B && n_qs < NC && data_ready(n_qs) && (n_qs == 0 || ready(B_ACCFREE, (n_qs & 1) ^ 1)) && ready(B_SBRDY, n_qs & 1)) {
          const uint64_t so = (uint64_t)(stage_of(n_qs) * STAGE16);
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < DK / 16; ++ks) umma_bf16(tm + tm_accv, d_kk + so + kstep(ks, 8192), d_gm + mstep(ks), ID_KG, ks > 0);
#pragma unroll
            for (int ks = 0; ks < DV / 16; ++ks) umma_bf16(tm + tm_acck, d_vk + so + kstep(ks, 8192), d_gk + kstep(ks, DK * 128), ID_VG, ks > 0);
            umma_commit(bar(B_SBFREE));
            FPB_TRACE(1, n_qs);
          }
          ++n_qs; progress = true;
        }
        // intra-chunk terms ACCV += P1 dOz, ACCK += P2 Q
        if (DO_B && n_pv < n_qs && ready(B_PRDY + (n_pv & 1), (n_pv >> 1) & 1)) {
          const uint64_t so = (uint64_t)(stage_of(n_pv) * STAGE16);
          const uint64_t po = (uint64_t)((n_pv & 1) * (G::P_BYTES >> 4));
          tc_fence_after();
          if (leader) {
#pragma unroll
            for (int ks = 0; ks < C / 16; ++ks) umma_bf16(tm + tm_accv, d_p1 + po + kstep(ks, 0), d_om + so + mstep(ks), ID_P1, 1);
#pragma unroll
            for (int ks = 0; ks < C / 16; ++ks) umma_bf16(tm + tm_acck, d_p2 + po + kstep(ks, 0), d_qm + so + mstep(ks), ID_P2, 1);
            umma_commit(bar(B_ACCFULL));
            FPB_TRACE(3, n_pv);
          }
          ++n_pv; progress = true;
          release();
        }
        release();      // (warp A may issue the scores of a chunk after its increment: nothing else would release then)
        if (progress) patience.progress();
        else if (__any_sync(0xffffffffu, patience.exhausted(abort_flag))) {
          if (leader) FPB_GIVE_UP((DO_A ? 0x200 : 0x500) | ((DO_A ? n_ds : n_pv) & 0xff));
          break;
        }
      }
      };
      if (!G::SPLIT) issue_loop(std::true_type{}, std::true_type{});
      else if (warp == 1) issue_loop(std::true_type{}, std::false_type{});
      else issue_loop(std::false_type{}, std::true_type{});
    }
  } else if (warp < STATE_WARP0) {                   // ---------------- score warps
    const int t = tid - SCORE_WARP0 * 32;            // 0..127
    const int q4 = warp & 3;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int r_lo = q4 * 16 + (lane >> 2);          // this thread's two rows of every M = 64 tile: r_lo, r_lo + 8
    const int cpair = (lane & 3) * 2;

    // one score tile -> upper-triangular (row j <= column i), times gamma^-L, bf16, swizzled K-major tile
    auto tile_to_p = [&](uint32_t taddr, uint8_t* pt, float cs) {
      uint32_t r[32];
      tmem_ld_16x256b_x8(tm + lane_base + taddr, r);
      tmem_wait_ld();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const int col = g * 8 + cpair;
        const float a0 = col >= r_lo ? __uint_as_float(r[4 * g]) * cs : 0.f;
        const float a1 = col + 1 >= r_lo ? __uint_as_float(r[4 * g + 1]) * cs : 0.f;
        const float b0 = col >= r_lo + 8 ? __uint_as_float(r[4 * g + 2]) * cs : 0.f;
        const float b1 = col + 1 >= r_lo + 8 ? __uint_as_float(r[4 * g + 3]) * cs : 0.f;
        *reinterpret_cast<uint32_t*>(pt + r_lo * 128 + ((g ^ (r_lo & 7)) << 4) + cpair * 2) = pack_bf16(a0, a1);
        *reinterpret_cast<uint32_t*>(pt + (r_lo + 8) * 128 + ((g ^ ((r_lo + 8) & 7)) << 4) + cpair * 2) = pack_bf16(b0, b1);
      }
    };
    auto make_p = [&](int n, int L) {
      tc_fence_after();
      const float cs = exp2f(-(float)L * lg);
      tile_to_p(tm_sc1(n), sm + G::OFF_P1 + (n & 1) * G::P_BYTES, cs);
      tile_to_p(tm_sc2(n), sm + G::OFF_P2 + (n & 1) * G::P_BYTES, cs);
      tc_fence_before();
      fence_async_smem();
      mbar_arrive(bar(B_PRDY + (n & 1)));
      if (t == 0) FPB_TRACE(7, n);
    };
    // one accumulator (64 x W) -> rows scaled by eta_j rs -> bf16 staging tile [W/64][64 rows][128 B] swizzled
    auto acc_to_staging = [&](uint32_t taddr, uint8_t* stg, int W, float z_lo, float z_hi, bool last) {
      for (int half = 0; half < W / 64; ++half) {
        uint32_t r[32];
        tmem_ld_16x256b_x8(tm + lane_base + taddr + half * 64, r);
        tmem_wait_ld();
        if (last && half == W / 64 - 1) { tc_fence_before(); mbar_arrive(bar(B_ACCFREE)); }
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t lo = pack_bf16(__uint_as_float(r[4 * g]) * z_lo, __uint_as_float(r[4 * g + 1]) * z_lo);
          const uint32_t hi = pack_bf16(__uint_as_float(r[4 * g + 2]) * z_hi, __uint_as_float(r[4 * g + 3]) * z_hi);
          *reinterpret_cast<uint32_t*>(stg + half * 8192 + r_lo * 128 + ((g ^ (r_lo & 7)) << 4) + cpair * 2) = lo;
          *reinterpret_cast<uint32_t*>(stg + half * 8192 + (r_lo + 8) * 128 + ((g ^ ((r_lo + 8) & 7)) << 4) + cpair * 2) = hi;
        }
      }
    };
    auto partial_store = [&](const uint8_t* stg, bf16* base, int64_t st_t, int W, Chunk ck) {
      for (int idx = t; idx < ck.L * (W / 8); idx += N_SCORE) {
        const int row = idx / (W / 8), ch = idx % (W / 8);
        const uint4 val = *reinterpret_cast<const uint4*>(stg + (ch >> 3) * 8192 + row * 128 + (((ch & 7) ^ (row & 7)) << 4));
        *reinterpret_cast<uint4*>(base + (int64_t)(ck.a + row) * st_t + ch * 8) = val;
      }
    };
    auto epilogue = [&](int n, Chunk ck, bool fail) -> bool {
      if (t == 0) tma_store_wait_read0();            // the previous stores have finished reading the staging tiles
      if (named_bar_or(1, N_SCORE, fail)) return false;
      if (t == 0) FPB_TRACE(9, n);
      tc_fence_after();
      const float z_lo = exp2f((float)(ck.L - 1 - r_lo) * lg) * rs, z_hi = exp2f((float)(ck.L - 9 - r_lo) * lg) * rs;
      acc_to_staging(tm_accv, sm + G::OFF_OUTV, DV, z_lo, z_hi, false);
      acc_to_staging(tm_acck, sm + G::OFF_OUTK, DK, z_lo, z_hi, true);
      const bool whole_box = ck.L == C || ck.a + ck.L >= p.T;
      if (whole_box) fence_async_smem();
      named_bar_sync(2, N_SCORE);
      if (whole_box) {
        if (t == 0) {
#pragma unroll
          for (int cb = 0; cb < DV / 64; ++cb) tma_store_4d(&p.map_dv, sbase + G::OFF_OUTV + cb * 8192, vcol + cb * 64, ck.a, h, b);
          if (dv_split) {
#pragma unroll
            for (int cb = 0; cb < DK / 64; ++cb) tma_reduce_add_4d(&p.map_dk, sbase + G::OFF_OUTK + cb * 8192, cb * 64, ck.a, h, b);
          } else {
#pragma unroll
            for (int cb = 0; cb < DK / 64; ++cb) tma_store_4d(&p.map_dk, sbase + G::OFF_OUTK + cb * 8192, cb * 64, ck.a, h, b);
          }
          tma_store_commit();
        }
      } else {   // chunk cut short by a block end: rows >= L belong to another chunk
        partial_store(sm + G::OFF_OUTV, p.dv_out + (int64_t)b * p.dv_sb + (int64_t)h * p.dv_sh, p.dv_st, DV, ck);
        partial_store(sm + G::OFF_OUTK, p.dk_out + (int64_t)b * p.dk_sb + (int64_t)h * p.dk_sh, p.dk_st, DK, ck);
      }
      if (t == 0) FPB_TRACE(10, n);
      return true;
    };

    if (NC > 0) {
      int n_p = 0, n_e = 0;
      Chunk ck_p = first, ck_e = first;
      Patience patience{0, 0};
      while (n_e < NC) {
        if (n_p < NC && n_p < n_e + G::NP && mbar_test_wait(bar(B_SCFULL + (n_p & 1)), (n_p >> 1) & 1)) {
          if (t == 0) FPB_TRACE(6, n_p);
          make_p(n_p, ck_p.L);
          ++n_p; prev_chunk(ck_p, p.block_size);
          patience.progress();
        } else if (n_e < n_p && mbar_test_wait(bar(B_ACCFULL), n_e & 1)) {
          if (t == 0) FPB_TRACE(8, n_e);
          if (!epilogue(n_e, ck_e, false)) break;
          ++n_e; prev_chunk(ck_e, p.block_size);
          patience.progress();
        } else if (patience.exhausted(abort_flag)) {
          FPB_GIVE_UP(0x300 | (n_e & 0xff));
          epilogue(n_e, ck_e, true);
          break;
        } else if (n_p < NC && n_p < n_e + G::NP) {
          mbar_try_wait_hint(bar(B_SCFULL + (n_p & 1)), (n_p >> 1) & 1, p.tune.idle_ns);
        } else {
          mbar_try_wait_hint(bar(B_ACCFULL), n_e & 1, p.tune.idle_ns);
        }
      }
      if (t == 0) tma_store_wait_all0();
    }
  } else if (warp < STATE_WARP0 + G::STATE_WARPS) {  // ---------------- state warps
    const int t = tid - STATE_WARP0 * 32;
    const int q4 = warp & 3;
    const int half = (warp - STATE_WARP0) >> 2;
    const uint32_t lane_base = (uint32_t)(q4 * 32) << 16;
    const int wcol0 = half * G::WCOLS;
    float S[G::NS];                                  // this thread's part of G (dk rows x dv columns)
    auto row_of = [&](int i) { return DK == 128 ? q4 * 32 + lane : q4 * 16 + (lane >> 2) + 8 * ((i >> 1) & 1); };
    auto col_of = [&](int i) { return DK == 128 ? wcol0 + i : wcol0 + 8 * (i >> 2) + 2 * (lane & 3) + (i & 1); };

    const int64_t state_elems = (int64_t)DK * p.dv;   // p.dv = DV, or 2 DV when two CTAs share a head
    // start: gradient of the returned state (none for suffix calls, whose end states are dropped);
    // end: dS_0, or for suffix m > 0 of a row the gradient of block state m-1
    const void* x_start = nullptr;
    void* x_end = nullptr;
    constexpr std::bool_constant<SF32> state_t{};
    constexpr std::true_type scratch_t{};
    constexpr int esz = SF32 ? 4 : 2;
    auto at = [&](const void* base, int64_t elems) { return (void*)((const char*)base + elems * esz); };
    // suffix calls: the batch index is (row, group of sfx_G consecutive suffixes); the walk goes through the group's
    // suffixes from the last to the first, and what it carries when it leaves suffix m is the gradient of the state
    // that suffix started from
    // (Grouping is compiled into the 64 x 64 kernel only - the shape suffixes come in; in the larger tiles its few
    // extra live registers spill the state, which costs the long-sequence workloads far more than grouping gains.)
    constexpr bool GROUPED = DK == 64 && DV == 64;
    const int sfx_g = GROUPED ? p.sfx_G : 1;
    const int groups = p.sfx_M > 0 ? p.sfx_M / sfx_g : 1;
    auto sfx_grad = [&](int m) -> void* {
      const int sfx_row = b / groups;
      if (m == 0) return p.g_end ? at(p.g_end, sfx_row * p.ge_sb + h * p.ge_sh) : nullptr;
      return p.sfx_blocks ? at(p.sfx_blocks, (((int64_t)sfx_row * p.sfx_N + (m - 1)) * p.H + h) * state_elems) : nullptr;
    };
    if (p.n_seg > 1) {
      // T-segments: G after this piece's last token was put into fp32 scratch by the scan; the first piece ends in dS_0
      x_start = p.seg_states + (((int64_t)b * p.H + h) * p.n_seg + seg) * state_elems;
      if (seg == 0 && p.g_end) x_end = at(p.g_end, b * p.ge_sb + h * p.ge_sh);
    } else if (p.sfx_M > 0) {
      if (sfx_g == 1) x_end = sfx_grad(b % groups);    // grouped walks store at every suffix start, inside the loop
    } else {
      if (p.g_start) x_start = at(p.g_start, b * p.gs_sb + h * p.gs_sh);
      if (p.g_end) x_end = at(p.g_end, b * p.ge_sb + h * p.ge_sh);
    }
    auto load_global = [&](const void* src_, auto f32, bool accumulate) {
      if constexpr (decltype(f32)::value) {
        const float* src = (const float*)src_ + vcol;
        if (DK == 128) {
          const float* rowp = src + (int64_t)row_of(0) * p.dv + wcol0;
#pragma unroll
          for (int i = 0; i < G::NS; i += 4) {
            const float4 val = *reinterpret_cast<const float4*>(rowp + i);
            S[i] = (accumulate ? S[i] : 0.f) + val.x; S[i + 1] = (accumulate ? S[i + 1] : 0.f) + val.y;
            S[i + 2] = (accumulate ? S[i + 2] : 0.f) + val.z; S[i + 3] = (accumulate ? S[i + 3] : 0.f) + val.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < G::NS; i += 2) {
            const float2 f = *reinterpret_cast<const float2*>(src + (int64_t)row_of(i) * p.dv + col_of(i));
            S[i] = (accumulate ? S[i] : 0.f) + f.x;
            S[i + 1] = (accumulate ? S[i + 1] : 0.f) + f.y;
          }
        }
      } else {
      const bf16* src = (const bf16*)src_ + vcol;
      if (DK == 128) {
        const bf16* rowp = src + (int64_t)row_of(0) * p.dv + wcol0;
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
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + (int64_t)row_of(i) * p.dv + col_of(i)));
          S[i] = (accumulate ? S[i] : 0.f) + f.x;
          S[i + 1] = (accumulate ? S[i + 1] : 0.f) + f.y;
        }
      }
      }
    };
    // POP: the gradient of a block state is added to G where the block ends.  Loaded at that moment into the register
    // layout of the state - 4-byte pieces, 512 sectors in flight per CTA - it stalled the walk's chunk-to-chunk chain for
    // a DRAM round trip and more (64 block ends per sequence cost the reverse walk 29 %).  The walk knows which block
    // comes next (the one before), so one thread fetches its gradient a block ahead with ONE TMA copy into shared
    // memory (a 64 x 64 tile, 128-byte swizzled: read back in the state's register layout - eight rows per warp
    // instruction - a plain row-major tile would put all eight on the same banks), and the addition reads it from there.
    // (The 64 x 64 instance with bf16 states - the POP shape; the others have no shared memory to spare.)
    constexpr bool PREFETCH = G::PF_BYTES > 0 && !SF32;
    int pf_blk = -1, pf_want = -1, pf_issued = 0, pf_taken = 0;
    auto block_grad = [&](int blk) { return at(p.block_grads, (((int64_t)b * p.n_blocks + blk) * p.H + h) * state_elems); };
    auto prefetch = [&](int blk) {
      if (t == 0) {
        // the buffer is free once every state thread has read the previous gradient out of it
        if (pf_issued > 0 && !mbar_wait(bar(B_PFFREE), (pf_issued - 1) & 1, abort_flag)) FPB_GIVE_UP(0x4fe);
        else {
          mbar_arrive_expect_tx(bar(B_PFFULL), G::PF_BYTES);
          tma_load_4d(sbase + G::OFF_PF, &p.map_bg, bar(B_PFFULL), 0, 0, blk * p.H + h, b);
        }
      }
      pf_blk = blk; ++pf_issued;
    };
    auto add_prefetched = [&]() {
      if (!mbar_wait(bar(B_PFFULL), (pf_issued - 1) & 1, abort_flag)) { FPB_GIVE_UP(0x4fd); return; }
      const uint8_t* src = sm + G::OFF_PF;             // [64 rows][128 B], 16-byte pieces XOR-swizzled by (row & 7)
#pragma unroll
      for (int i = 0; i < G::NS; i += 2) {
        const int row = row_of(i), col = col_of(i);
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src + row * 128 + (((col >> 3) ^ (row & 7)) << 4) + (col & 7) * 2));
        S[i] += f.x; S[i + 1] += f.y;
      }
      mbar_arrive(bar(B_PFFREE));
      ++pf_taken;
    };
    auto inject = [&](int end) {
      if (p.block_size > 0 && p.block_grads && end % p.block_size == 0 && end / p.block_size - 1 < p.n_blocks) {
        const int blk = end / p.block_size - 1;
        if (PREFETCH && pf_blk == blk) add_prefetched();
        else load_global(block_grad(blk), state_t, true);
        // the walk's next block end, going down: the start of this block, if this CTA's piece reaches below it.  The
        // fetch is issued after the state copy that follows (thread 0 first waits for the other warps to have read the
        // buffer: better while the walk waits for the next increment than in front of the copy).
        if (PREFETCH && blk > 0 && (int64_t)blk * p.block_size > t0) pf_want = blk - 1;
      }
    };
    auto store_global = [&](void* dst_) {
      if constexpr (SF32) {
        float* dst = (float*)dst_ + vcol;
        if (DK == 128) {
          float* rowp = dst + (int64_t)row_of(0) * p.dv + wcol0;
#pragma unroll
          for (int i = 0; i < G::NS; i += 4) *reinterpret_cast<float4*>(rowp + i) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < G::NS; i += 2)
            *reinterpret_cast<float2*>(dst + (int64_t)row_of(i) * p.dv + col_of(i)) = make_float2(S[i], S[i + 1]);
        }
      } else {
      bf16* dst = (bf16*)dst_ + vcol;
      if (DK == 128) {
        bf16* rowp = dst + (int64_t)row_of(0) * p.dv + wcol0;
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
          *reinterpret_cast<uint32_t*>(dst + (int64_t)row_of(i) * p.dv + col_of(i)) = pack_bf16(S[i], S[i + 1]);
      }
      }
    };
    // Gb: [DV/64 column blocks][DK rows][128 bytes], 16-byte pieces XOR-swizzled by (row & 7): an MN-major B
    // operand for K Gb and a K-major B operand for V Gb^T
    auto publish_gb = [&]() {
      uint8_t* gb = sm + G::OFF_GB;
      if (DK == 128) {
        const int row = row_of(0);
#pragma unroll
        for (int i = 0; i < G::NS; i += 8) {
          const int col = col_of(i);
          uint4 val;
          val.x = pack_bf16(S[i], S[i + 1]); val.y = pack_bf16(S[i + 2], S[i + 3]);
          val.z = pack_bf16(S[i + 4], S[i + 5]); val.w = pack_bf16(S[i + 6], S[i + 7]);
          *reinterpret_cast<uint4*>(gb + (col >> 6) * (DK * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4)) = val;
        }
      } else {
#pragma unroll
        for (int i = 0; i < G::NS; i += 2) {
          const int row = row_of(i), col = col_of(i);
          *reinterpret_cast<uint32_t*>(gb + (col >> 6) * (DK * 128) + row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4) + (col & 7) * 2) =
              pack_bf16(S[i], S[i + 1]);
        }
      }
      fence_async_smem();
      mbar_arrive(bar(B_SBRDY));
    };
    // dOz = zeta . dO in place (rows >= L zeroed)
    auto scale_do = [&](int n, int L) {
      const int s = stage_of(n);
      uint8_t* vt = sm + G::OFF_STAGE + s * G::STAGE_BYTES + G::OFF_DO;
      for (int idx = t; idx < C * DV / 8; idx += G::N_STATE) {
        const int row = (idx >> 3) & 63;
        uint4* ptr = reinterpret_cast<uint4*>(vt + idx * 16);
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (row < L) {
          const float e = exp2f((float)(row + 1) * lg);
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
      fence_async_smem();
      mbar_arrive(bar(B_VRDY + s));
    };

    if (x_start) {
      if (p.n_seg > 1) load_global(x_start, scratch_t, false);
      else load_global(x_start, state_t, false);
    }
    else {
#pragma unroll
      for (int i = 0; i < G::NS; ++i) S[i] = 0.f;
    }
    if (NC > 0) {
      int n_v = 0, n_u = 0;
      bool publish_due = true;
      Chunk ck_v = first, ck_u = first;
      inject(first.a + first.L);
      Patience patience{0, 0};
      while (n_u < NC) {
        bool progress = false;
        if (n_v < NC && mbar_test_wait(bar(B_FULL + stage_of(n_v)), stage_ph(n_v))) {
          scale_do(n_v, ck_v.L);
          if (t == 0) FPB_TRACE(11, n_v);
          ++n_v; prev_chunk(ck_v, p.block_size);
          progress = true;
        }
        if (publish_due) {
          if (n_u == 0 || mbar_test_wait(bar(B_SBFREE), (n_u - 1) & 1)) {
            publish_gb();
            if (t == 0) FPB_TRACE(13, n_u);
            publish_due = false; progress = true;
            if (PREFETCH && pf_want >= 0) { prefetch(pf_want); pf_want = -1; }
          }
        } else if (mbar_test_wait(bar(B_DSFULL + (n_u & 1)), (n_u >> 1) & 1)) {
          if (t == 0) FPB_TRACE(12, n_u);
          tc_fence_after();
          const float gl = exp2f((float)ck_u.L * lg);
#pragma unroll
          for (int i0 = 0; i0 < G::NS; i0 += 16) {
            uint32_t r[16];
            if (DK == 128) tmem_ld_32x32b_x16(tm + lane_base + tm_dg(n_u) + wcol0 + i0, r);
            else tmem_ld_16x256b_x4(tm + lane_base + tm_dg(n_u) + wcol0 + i0 * 2, r);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) S[i0 + i] = fmaf(gl, S[i0 + i], __uint_as_float(r[i]));
          }
          tc_fence_before();
          mbar_arrive(bar(B_DSFREE + (n_u & 1)));
          ++n_u;
          if (GROUPED && sfx_g > 1 && ck_u.a % p.block_size == 0) {   // that was the first chunk of a suffix
            void* dst = sfx_grad((b % groups) * sfx_g + ck_u.a / p.block_size);
            if (dst) store_global(dst);
#pragma unroll
            for (int i = 0; i < G::NS; ++i) S[i] = 0.f;      // the suffix before it ends in a state nobody reads
          }
          if (n_u < NC) {
            prev_chunk(ck_u, p.block_size);
            inject(ck_u.a + ck_u.L);
            publish_due = true;
          }
          progress = true;
        }
        if (progress) patience.progress();
        else if (patience.exhausted(abort_flag)) { FPB_GIVE_UP(0x400 | (n_u & 0xff)); break; }
        else if (publish_due) mbar_try_wait_hint(bar(B_SBFREE), (n_u - 1) & 1, p.tune.idle_ns);
        else mbar_try_wait_hint(bar(B_DSFULL + (n_u & 1)), (n_u >> 1) & 1, p.tune.idle_ns);
      }
    }
    if (x_end && !*abort_flag) store_global(x_end);
    if (PREFETCH && t == 0 && pf_issued > pf_taken) {      // (only after a give-up) let the copy in flight land
      const long long w0 = clock64();
      while (!mbar_try_wait(bar(B_PFFULL), (pf_issued - 1) & 1) && clock64() - w0 < wait_limit(abort_flag)) {}
    }
  }

  // ---------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tm, G::TM_COLS); }
}

template <int DK, int DV, bool SF32>
int launch_fused_t(const BwdParams& p, dim3 grid, cudaStream_t stream) {
  using G = BCfg<DK, DV>;
  static std::atomic<bool> configured[64];
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || !configured[dev].load(std::memory_order_acquire)) {
    if (cudaFuncSetAttribute(bwd_fused_kernel<DK, DV, SF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, G::SMEM) != cudaSuccess)
      return FPB_ERR_LAUNCH;
    if (dev >= 0 && dev < 64) configured[dev].store(true, std::memory_order_release);
  }
  bwd_fused_kernel<DK, DV, SF32><<<grid, G::NTHREADS, G::SMEM, stream>>>(p);
  return FPB_OK;
}

bool state_ok(const StateView& s, bool f32) {
  const int64_t m = f32 ? 4 : 8;
  return !s.data || ((uintptr_t)s.data % 16 == 0 && s.sb % m == 0 && s.sh % m == 0);
}
int gcd_int(int a, int b) { while (b) { const int t = a % b; a = b; b = t; } return a; }

}  // namespace

// dK, dV and dS_0 in one reverse walk.  FPB_UMMA_NOT_APPLICABLE when the shape is not one the kernel is built for.
int launch_bwd_fused(const UmmaBwdArgs& a, cudaStream_t stream, int* n_launched) {
  // dv = 256 next to dk = 128: two CTAs per head, one per half of dv, on the 128 x 128 instance.  Each writes its half
  // of dV and of dS_0; dK is the sum of the two CTAs' partial results, which TMA adds to the zeroed tensor in L2.  Only
  // where every chunk is stored as a whole tile (no POP blocks, no suffixes).
  const bool dv_halves = a.dk == 128 && a.dv == 256 && a.block_size == 0 && a.sfx_grad.M == 0 && col_split_enabled();
  const bool dims_ok = ((a.dk == 64 || a.dk == 128) && (a.dv == 64 || a.dv == 128)) || dv_halves;
  if (!dims_ok || a.dtype != FPB_BF16 || a.T <= 0 || a.B > 65535 || a.H > 65535) return FPB_UMMA_NOT_APPLICABLE;
  if (!tma_addressable(a.q, 2) || !tma_addressable(a.k, 2) || !tma_addressable(a.v, 2) || !tma_addressable(a.dO, 2) ||
      !tma_addressable(a.dK, 2) || !tma_addressable(a.dV, 2))
    return FPB_UMMA_NOT_APPLICABLE;
  if (!state_ok(a.d_s_out, a.state_f32) || !state_ok(a.d_s0, a.state_f32) || (uintptr_t)a.d_block_states % 16 ||
      (uintptr_t)a.sfx_grad.blocks % 16)
    return FPB_UMMA_NOT_APPLICABLE;
  BwdParams p;
  int r;
  int B = a.B, T = a.T, block_size = a.block_size;
  const int H = a.H;
  // suffix calls: G consecutive suffixes of a row as one sequence per CTA (see launch_one in retention_scan_sm100.cu)
  SeqView q = a.q, k = a.k, v = a.v, dO = a.dO, dK = a.dK, dV = a.dV;
  int G = 1;
  if (a.sfx_grad.M > 1 && a.block_size == 0) {
    bool contiguous = true;
    for (const SeqView* s : {&q, &k, &v, &dO, &dK, &dV}) contiguous = contiguous && s->sb == (int64_t)T * s->st;
    if (contiguous && a.dk == 64 && a.dv == 64) G = choose_suffix_group(a.sfx_grad.M, (long long)(B / a.sfx_grad.M) * H);
    if (G > 1) {
      B /= G; block_size = T; T *= G;
      for (SeqView* s : {&q, &k, &v, &dO, &dK, &dV}) s->sb *= G;
    }
  }
  // under-filled: cut the sequences into T-segments (segment_scan.cu) - local values of G per piece from a reverse
  // state-only walk over (Q, dO), the scan (which also writes dS_0), then this kernel once per piece
  Segments sg{1, 0};
  if (segments_enabled() && a.scratch && a.sfx_grad.M == 0) {
    const int align = a.block_size > 0 ? C / gcd_int(C, a.block_size) * a.block_size : C;
    sg = choose_segments((long long)H * B * (dv_halves ? 2 : 1), 1, T, align, (long long)B * H, (long long)a.dk * a.dv, a.scratch_bytes, B);
  }
  if (sg.n > 1) {
    if ((r = launch_segment_states(a.q, a.dO, true, a.d_block_states, a.gamma, B, T, H, a.dk, a.dv, a.block_size, a.n_blocks,
                                   a.state_f32, sg, a.scratch, stream)) != FPB_OK)
      return r;
    if ((r = launch_segment_combine(a.scratch, sg, B, T, H, a.dk, a.dv, a.gamma, true, a.d_s_out, a.state_f32, stream)) != FPB_OK)
      return r;
    *n_launched += 2;
  }
  if ((r = make_seq_map(&p.map_q, q, B, T, H, a.dk, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_k, k, B, T, H, a.dk, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_v, v, B, T, H, a.dv, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_do, dO, B, T, H, a.dv, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_dk, dK, B, T, H, a.dk, C)) != FPB_OK) return r;
  if ((r = make_seq_map(&p.map_dv, dV, B, T, H, a.dv, C)) != FPB_OK) return r;
  if (a.dk == 64 && a.dv == 64 && !a.state_f32 && a.d_block_states && a.n_blocks > 0) {
    // (B, N, H, dk, dv) contiguous as a 4-D tensor of 64-wide rows: dk rows per (block, head), N * H of those per batch row
    const SeqView bg{const_cast<void*>(a.d_block_states), (int64_t)a.n_blocks * H * a.dk * a.dv, (int64_t)a.dv, (int64_t)a.dk * a.dv};
    if ((r = make_seq_map(&p.map_bg, bg, B, a.dk, a.n_blocks * H, a.dv, C)) != FPB_OK) return r;
  }
  p.dk_out = (bf16*)dK.data; p.dk_sb = dK.sb; p.dk_st = dK.st; p.dk_sh = dK.sh;
  p.dv_out = (bf16*)dV.data; p.dv_sb = dV.sb; p.dv_st = dV.st; p.dv_sh = dV.sh;
  const bool split = sg.n > 1;
  p.g_start = split ? nullptr : a.d_s_out.data; p.gs_sb = a.d_s_out.sb; p.gs_sh = a.d_s_out.sh;
  p.g_end = a.d_s0.data; p.ge_sb = a.d_s0.sb; p.ge_sh = a.d_s0.sh;      // split: written by the piece the walk reaches last
  p.block_grads = a.d_block_states;
  p.sfx_blocks = a.sfx_grad.blocks; p.sfx_M = a.sfx_grad.M; p.sfx_N = a.sfx_grad.N; p.sfx_G = G;
  p.T = T; p.H = H; p.dk = a.dk; p.dv = a.dv; p.block_size = block_size; p.n_blocks = a.n_blocks;
  p.state_f32 = a.state_f32 ? 1 : 0;
  p.n_seg = sg.n; p.seg_len = sg.seg_len; p.seg_states = a.scratch;
  p.tune = walk_tuning();
  p.status = device_status_ptr();
  p.trace = debug_trace_ptr();
  if (!p.status) return FPB_ERR_LAUNCH;
  for (int h = 0; h < H; ++h) p.log2g[h] = (float)std::log2((double)a.gamma[h]);
  const dim3 grid(dv_halves ? 2 : 1, H, B * sg.n);
  if (dv_halves) {
    launch_zero_seq(dK, B, T, H, a.dk, stream);
    ++*n_launched;
  }
  const int tile_dv = dv_halves ? 128 : a.dv;
#define FPB_FUSED_CASE(DK_, DV_) \
  if (a.dk == DK_ && tile_dv == DV_) r = a.state_f32 ? launch_fused_t<DK_, DV_, true>(p, grid, stream) : launch_fused_t<DK_, DV_, false>(p, grid, stream)
  r = FPB_ERR_BAD_SHAPE;
  FPB_FUSED_CASE(128, 128); FPB_FUSED_CASE(64, 64); FPB_FUSED_CASE(64, 128); FPB_FUSED_CASE(128, 64);
#undef FPB_FUSED_CASE
  if (r == FPB_OK) ++*n_launched;
  return r;
}

}  // namespace fpb
