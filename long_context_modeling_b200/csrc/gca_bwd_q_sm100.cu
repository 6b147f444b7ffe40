// GCA backward, q-major pass (dQ, dw and the per-row terms the kv-major pass needs) on tcgen05 /
// TMEM / TMA, bf16, S = L = D = 64.
//
// Unit = (sequence n, query chunk j, PAIR of q heads) as in the forward: Q and dO of the unit stay
// in shared memory while the K retrieved slots stream through.  Per slot the kernel recomputes
// S = Q K_k^T  and  dP = dO V_k^T;  one thread per query row forms  P = exp2(S c - LSE),
// Di = rowsum(P * dP)  (which replaces the reference's extra o = v^T p^T product,
// ltriton/gca.py:382)  and  dS = w P (dP - Di);  dQ += dS K_k  accumulates over the slots in tensor
// memory, and the per-head parts of  dw_k = sum_rows Di  go to a partials buffer that a tiny
// fixed-order kernel reduces.  For every (row, slot) the two per-row terms of the kv-major pass,
// (log2|w| - LSE) / c and -Di, are also written to the workspace, each split into three bf16
// values: the kv-major pass (gca_bwd_kv_sm100.cu), which runs AFTER this one, adds them to its
// recomputed scores with one extra MMA K step (the reference hands Di from one of its two kernels
// to the other in the same way, ltriton/gca.py:385,459).
//
// Every product is computed per head with 64-row MMAs.  A 64-row accumulator or tensor-memory
// operand occupies lanes 0-15 of every 32-lane quarter, so head B's tiles, placed at lane offset
// 16, share head A's columns: S and dP of a head PAIR take 128 columns, and THREE such score
// buffers plus two dQ accumulators (64 columns each for both heads) fill the 512 columns.  A
// buffer goes through  MMA (S, dP) -> worker -> MMA (dQ) -> release  in a few thousand cycles;
// with three of them, and one worker warpgroup per buffer, slot g + 1 and g + 2 are computed while
// slot g is still being worked on.  (With stacked 128-row products S and dP took 256 columns and
// could not be double-buffered: issue of the eight MMAs, the workers' read and two barrier hops
// formed a serial chain of ~1,900 cycles per slot.)
//
// A worker thread never holds a whole row in registers: it walks its 64 keys twice in passes of
// 16 columns.  Pass 1 reads S and dP, accumulates Di and writes P as packed bf16 over the S
// columns it has already read; pass 2 reads P and dP back and writes dS = P (w dP - w Di) as
// packed bf16 over the dP columns, from where the dQ product takes it as its A operand (lane =
// row of A = query row).  82 registers instead of 161, which is what lets three worker groups
// and twenty warps fit.  Shared memory sees only the TMA copies and the MMAs' operand reads.
//
// CTA = 20 warps: three worker warpgroups, one TMA producer, three MMA issuers (S, dP, dQ), and a
// warpgroup that writes the finished dQ tiles.  No
// atomics: gradients are bit-reproducible.  Every wait is bounded (GCA_STATUS_TIMEOUT on expiry).
#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace gca {

long long* profile_buffer();

namespace {

using namespace sm100;

constexpr int TILE_BYTES = 64 * 64 * 2;
constexpr int PAIR_BYTES = 2 * TILE_BYTES;
constexpr uint32_t PAIR16 = PAIR_BYTES >> 4, TILE16 = TILE_BYTES >> 4;
#ifndef GCA_Q_NBUF
#define GCA_Q_NBUF 3
#endif
constexpr int NBUF = GCA_Q_NBUF;
static_assert(NBUF == 2 || NBUF == 3, "score buffers");
// One issuing warp per product.  An issuer needs ~1,300 cycles per slot (probe of its two barriers
// ~330, eight 64-row MMAs and the commits ~600, loop bookkeeping ~300: event traces), which is what
// bounds the kernel today; yet more issuing warps were measured SLOWER, both ways tried: one warp
// per head (the heads of a slot share the buffer's columns) 0.835 against 0.567 ms, one warp per
// slot parity for S and dP 1,640 against 1,390 cycles per slot -- every extra polling warp slows
// the shared-memory path that the MMAs' operand reads already load to ~875 of those cycles.
// Worker warpgroups: slot g goes to group g % NWG (and to buffer g % NBUF).
#ifndef GCA_Q_NWG
#define GCA_Q_NWG GCA_Q_NBUF
#endif
constexpr int NWG = GCA_Q_NWG;              // measured: 2 groups 0.653 ms, 3 groups 0.55-0.57 ms
static_assert(NWG >= 2 && NWG <= NBUF, "worker groups");
// The issuers probe the NEXT slot's barriers before they issue the current slot's MMAs, so that the
// probes' shared-memory round trip runs under the issue: 0.562 -> 0.538 ms.  (The same in the
// forward and in the kv-major kernel was measured slower: 0.434 against 0.414 and 0.634 against
// 0.613 ms.)
#ifndef GCA_Q_PREPROBE
#define GCA_Q_PREPROBE 1
#endif
constexpr int PROD_WARP = 4 * NWG, ISSUE_S = PROD_WARP + 1, ISSUE_DP = ISSUE_S + 1, ISSUE_DQ = ISSUE_DP + 1;
constexpr int WRITER_WARP = (ISSUE_DQ + 1 + 3) / 4 * 4;   // a multiple of 4: warp % 4 = its TMEM lane quarter
constexpr int NTHREADS = (WRITER_WARP + 4) * 32;
constexpr int TMEM_COLS = 512;
constexpr uint32_t LANE16 = 16u << 16;            // TMEM lane offset of head B's 64-row tile
constexpr uint32_t IDESC_64 = umma_idesc_bf16(64, 64, 0, 0);
constexpr uint32_t IDESC_DQ = umma_idesc_bf16(64, 64, 0, 1);       // A: tensor memory, B: MN-major
constexpr int STEP_K = 2;      // K-major operand: +32 bytes (>> 4) per K step of 16
constexpr int STEP_MN = 128;   // MN-major operand: +2048 bytes (>> 4) per K step of 16

#ifndef GCA_Q_NKS
#define GCA_Q_NKS 6
#endif
#ifndef GCA_Q_NVS
#define GCA_Q_NVS 4
#endif
constexpr int NKS = GCA_Q_NKS, NVS = GCA_Q_NVS;
constexpr int OFF_QDO = 0;                                   // [2][Q pair | dO pair]
constexpr int OFF_K = OFF_QDO + 2 * 2 * PAIR_BYTES;          // [NKS][K pair]
constexpr int OFF_V = OFF_K + NKS * PAIR_BYTES;              // [NVS][V pair]
constexpr int OFF_BAR = OFF_V + NVS * PAIR_BYTES;
constexpr int OFF_IDX = OFF_BAR + 512;
constexpr int SMEM_BYTES = OFF_IDX + 256 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
enum Bar { QDO_FULL = 0, QDO_EMPTY = 2, K_FULL = 4, K_EMPTY = K_FULL + NKS, V_FULL = K_EMPTY + NKS,
           V_EMPTY = V_FULL + NVS, SP_FULL = V_EMPTY + NVS, PDS_FULL = SP_FULL + NBUF, BUF_FREE = PDS_FULL + NBUF,
           ACC_FULL = BUF_FREE + NBUF, ACC_EMPTY = ACC_FULL + 2, NUM_BARS = ACC_EMPTY + 2 };
static_assert(NUM_BARS * 8 + 16 <= 512, "barrier block");
// Tensor-memory columns.  Buffer b (slot g uses b = g % NBUF) = 128 columns: S at +0 and dP at
// +64 as float32; afterwards P at +0 and dS at +64 as packed bf16 (32 columns each).  Behind the
// buffers two dQ accumulators of 64 columns (unit u uses accumulator u % 2).
constexpr uint32_t BUF_COLS = 128, COL_DPT = 64, COL_DQ = NBUF * BUF_COLS;
static_assert(NBUF * BUF_COLS + 128 <= TMEM_COLS, "tensor memory");

// x as the sum of three bf16 values (24 mantissa bits: float32 precision).
__device__ __forceinline__ void split3(float x, __nv_bfloat16& h, __nv_bfloat16& m, __nv_bfloat16& l) {
  h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);
  m = __float2bfloat16_rn(r1);
  l = __float2bfloat16_rn(r1 - __bfloat162float(m));
}
// The 16-byte record of one (query row, slot) for the kv-major pass: see BwdQParams::rowterm.
__device__ __forceinline__ uint4 row_terms(float a, float b) {
  __nv_bfloat16 a0, a1, a2, b0, b1, b2;
  split3(a, a0, a1, a2);
  split3(b, b0, b1, b2);
  auto pk = [](__nv_bfloat16 lo, __nv_bfloat16 hi) {
    return (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
  };
  return make_uint4(pk(a0, a1), pk(a2, b0), pk(b1, b2), 0u);
}
// log2|w|, kept finite: a weight of zero becomes 2^-200, which the exponential flushes to zero.
__device__ __forceinline__ float log2_abs_clamped(float w) {
  const float a = fabsf(w);
  return a > 0.f ? fmaxf(__log2f(a), -200.f) : -200.f;
}

__device__ __forceinline__ void drain(uint64_t* bars, int full0, uint32_t issued, int depth) {
  for (uint32_t back = 0; back < (uint32_t)depth && back < issued; ++back) {
    const uint32_t g = issued - 1 - back;
    for (int i = 0; i < (1 << 20); ++i)
      if (mbar_try_wait(&bars[full0 + g % depth], (g / depth) & 1)) break;
  }
}

struct BwdQParams {
  CUtensorMap tm_q, tm_do, tm_k2, tm_v2, tm_k1, tm_v1;
  const int32_t* indices;
  const float* weights;
  const float* lse;
  __nv_bfloat16* dq;
  float* dw_part;           // (N*J, Hq, K, 4): one partial per (row block, head, slot, 16-row quarter)
  uint4* rowterm;           // (N*J, Hq, K, 64) x 16 bytes: per (row block, head, slot, query row) eight bf16 values
                            // (a0, a1, a2, b0, b1, b2, 0, 0) with a0 + a1 + a2 = (log2|w| - lse) / c2 and
                            // b0 + b1 + b2 = -Di: the kv-major pass adds them to its scores with one MMA K step
  float inv_c2;
  int32_t* status;
  long long* prof;
  long long dqs[4];
  int units;
  int N, J, Hq, Hkv, G, K, C, HP;
  int wide_store;           // dq rows are 32-byte aligned: 256-bit stores
  float c2, sm_scale;
};

// Heads of a unit: q heads h0, h0 + 1; their kv heads are hk0 and hk0 + 1, or both hk0 (`share`,
// grouped-query attention: one K / V tile serves both).
struct QInfo { int h0, hk0; bool two, share; };
__device__ __forceinline__ QInfo q_info(const BwdQParams& p, int hp) {
  QInfo t;
  t.h0 = 2 * hp;
  t.two = (t.h0 + 1) < p.Hq;
  if (p.G == 1) { t.hk0 = t.h0; t.share = false; }
  else { t.hk0 = t.h0 / p.G; t.share = t.two && ((t.h0 + 1) / p.G == t.hk0); }
  return t;
}
__device__ __forceinline__ int q_load_row(const BwdQParams& p, int u, int zj, int lane) {
  if (u >= p.units || lane >= p.K) return -1;
  return p.indices[(long long)zj * p.K + lane];
}
__device__ __forceinline__ unsigned q_valid(const BwdQParams& p, int idx) {
  return __ballot_sync(0xffffffffu, idx >= 0 && idx < p.C);
}

// One lane: Q + dO per unit, K and V per slot.
__device__ void q_producer(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane) {
  int* sidx = reinterpret_cast<int*>(smem + OFF_IDX);
  PairCursor c;
  c.init(p.HP);
  Ring rk, rv; rk.init(NKS); rv.init(NVS);
  uint32_t ucnt = 0, issued = 0;
  bool ok = true;
  int next_idx = q_load_row(p, c.u, c.outer, lane);
  for (; c.u < p.units; c.advance()) {
    const int my_idx = next_idx;
    next_idx = q_load_row(p, c.u + gridDim.x, c.next_outer(), lane);
    const unsigned mask = q_valid(p, my_idx);
    if (mask == 0) continue;
    __syncwarp();
    sidx[lane] = my_idx;
    __syncwarp();
    const uint32_t un = ucnt++;
    if (lane != 0 || !ok) continue;
    const QInfo t = q_info(p, c.inner);
    const int n = c.outer / p.J, j = c.outer - n * p.J;
    {
      const uint32_t ub = un & 1;
      ok = mbar_wait_bounded(&bars[QDO_EMPTY + ub], ((un >> 1) & 1) ^ 1, abort_flag);
      if (!ok) continue;
      uint8_t* base = smem + OFF_QDO + ub * 2 * PAIR_BYTES;
      mbar_arrive_expect_tx(&bars[QDO_FULL + ub], 2 * PAIR_BYTES);
      tma_load_5d(base, &p.tm_q, &bars[QDO_FULL + ub], 0, 0, t.h0, j, n);
      tma_load_5d(base + PAIR_BYTES, &p.tm_do, &bars[QDO_FULL + ub], 0, 0, t.h0, j, n);
    }
    const CUtensorMap* tmk = t.share ? &p.tm_k1 : &p.tm_k2;
    const CUtensorMap* tmv = t.share ? &p.tm_v1 : &p.tm_v2;
    const uint32_t bytes = t.share ? TILE_BYTES : PAIR_BYTES;
    for (unsigned m = mask; m; m &= m - 1) {
      const int idx = sidx[__ffs(m) - 1];
      ok = mbar_wait_bounded(&bars[K_EMPTY + rk.st], rk.ph ^ 1, abort_flag);
      if (!ok) break;
      mbar_arrive_expect_tx(&bars[K_FULL + rk.st], bytes);
      tma_load_5d(smem + OFF_K + rk.st * PAIR_BYTES, tmk, &bars[K_FULL + rk.st], 0, 0, t.hk0, idx, n);
      rk.next();
      ok = mbar_wait_bounded(&bars[V_EMPTY + rv.st], rv.ph ^ 1, abort_flag);
      if (!ok) break;
      mbar_arrive_expect_tx(&bars[V_FULL + rv.st], bytes);
      tma_load_5d(smem + OFF_V + rv.st * PAIR_BYTES, tmv, &bars[V_FULL + rv.st], 0, 0, t.hk0, idx, n);
      rv.next();
      ++issued;
    }
  }
  if (lane == 0 && *abort_flag) {
    drain(bars, K_FULL, issued, NKS);
    drain(bars, V_FULL, issued, NVS);
    drain(bars, QDO_FULL, ucnt, 2);
  }
}

// role 0: S per slot;  role 1: dP per slot;  role 2: dQ += dS K per slot.  All 32 lanes run this
// code; elect.sync inside the MMA / commit wrappers picks the issuing lane.
template <int ROLE>
__device__ void q_issuer(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                         uint32_t tmem_base) {
  const uint64_t dQDO = umma_desc_sw128(smem_u32(smem + OFF_QDO));
  const uint64_t dK = umma_desc_sw128(smem_u32(smem + OFF_K)), dV = umma_desc_sw128(smem_u32(smem + OFF_V));
  const uint64_t dKmn = umma_desc_sw128_mn_blocks(smem_u32(smem + OFF_K), TILE_BYTES);
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(ROLE == 1 ? NVS : NKS);
  uint32_t ucnt = 0, g = 0;
  uint32_t b = 0, bph = 0;                                // g % NBUF and the parity of g / NBUF
  bool ok = true;
  int next_idx = q_load_row(p, c.u, c.outer, lane);
  for (; c.u < p.units && ok; c.advance()) {
    const int my_idx = next_idx;
    next_idx = q_load_row(p, c.u + gridDim.x, c.next_outer(), lane);
    const unsigned mask = q_valid(p, my_idx);
    if (mask == 0) continue;
    const uint32_t un = ucnt++;
    const int nv = __popc(mask);
    const QInfo t = q_info(p, c.inner);
    const uint32_t ub = un & 1, uph = (un >> 1) & 1;
    const uint32_t kt1 = t.share ? 0u : TILE16;            // head B's K / V tile inside the stage
    if (ROLE != 2) ok = mbar_wait_warp(&bars[QDO_FULL + ub], uph, abort_flag, lane);
    else ok = mbar_wait_warp(&bars[ACC_EMPTY + ub], uph ^ 1, abort_flag, lane);
    bool pre_a = false, pre_b = false;           // early probe results for the coming slot
    for (int i = 0; i < nv && ok; ++i, ++g) {
      const uint32_t tbuf = tmem_base + b * BUF_COLS;
      if (ROLE != 2) {
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 0, g);
        // the tile has landed AND the buffer's previous contents (the packed dS of slot g - NBUF)
        // have been consumed: both barriers are probed at once (one shared-memory round trip)
        // (probed while the previous slot's MMAs were being issued, when there was one in this unit)
        ok = mbar_wait_warp2_probed(&bars[(ROLE == 0 ? K_FULL : V_FULL) + ring.st], ring.ph, pre_a, &bars[BUF_FREE + b], bph ^ 1,
                                    pre_b, abort_flag);
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 3, g);
        if (!ok) break;
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 1, g);
        tc_fence_after();
        pre_a = pre_b = false;
        if (GCA_Q_PREPROBE && i + 1 < nv) {              // the next slot's two barriers
          const uint32_t nst = ring.st + 1 == (uint32_t)ring.depth ? 0u : ring.st + 1, nph = nst ? ring.ph : ring.ph ^ 1;
          const uint32_t nb = b + 1 == NBUF ? 0u : b + 1, nbph = nb ? bph : bph ^ 1;
          pre_a = mbar_test_wait(&bars[(ROLE == 0 ? K_FULL : V_FULL) + nst], nph);
          pre_b = mbar_test_wait(&bars[BUF_FREE + nb], nbph ^ 1);
        }
        const uint64_t a = dQDO + ub * 2 * PAIR16 + (ROLE == 0 ? 0u : PAIR16);          // Q pair | dO pair
        const uint64_t bt = (ROLE == 0 ? dK : dV) + ring.st * PAIR16;
        const uint32_t d = tbuf + (ROLE == 0 ? 0u : COL_DPT);
#pragma unroll
        for (int tl = 0; tl < 2; ++tl) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ss_elect(d + (tl ? LANE16 : 0u), a + tl * TILE16 + kk * STEP_K, bt + (tl ? kt1 : 0u) + kk * STEP_K,
                               IDESC_64, (uint32_t)(kk > 0));
        }
        umma_commit_elect(&bars[SP_FULL + b]);            // the barrier expects both the S and the dP commit
        if (ROLE == 1) umma_commit_elect(&bars[V_EMPTY + ring.st]);
        if (i == nv - 1) umma_commit_elect(&bars[QDO_EMPTY + ub]);    // expects both issuers' commits
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 2, g);
      } else {
        ok = mbar_wait_warp2_probed(&bars[PDS_FULL + b], bph, pre_a, &bars[PDS_FULL + b], bph, true, abort_flag);
        if (!ok) break;
        if (lane == 0) GCA_TRACE_BUF(p.prof, 5, g);
        tc_fence_after();
        pre_a = false;
        if (GCA_Q_PREPROBE && i + 1 < nv) {
          const uint32_t nb = b + 1 == NBUF ? 0u : b + 1, nbph = nb ? bph : bph ^ 1;
          pre_a = mbar_test_wait(&bars[PDS_FULL + nb], nbph);
        }
        // dQ += dS K_k per head: A = dS from tensor memory (lane = query row, 8 columns per K step
        // of 16 keys), B = the head's K tile read N-contiguous (MN-major)
        const uint32_t acc = tmem_base + COL_DQ + ub * 64;
        const uint64_t bk = dKmn + ring.st * PAIR16;
#pragma unroll
        for (int tl = 0; tl < 2; ++tl) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ts_elect(acc + (tl ? LANE16 : 0u), tbuf + COL_DPT + (tl ? LANE16 : 0u) + kk * 8,
                               bk + (tl ? kt1 : 0u) + kk * STEP_MN, IDESC_DQ, (uint32_t)(i > 0 || kk > 0));
        }
        umma_commit_elect(&bars[BUF_FREE + b]);
        umma_commit_elect(&bars[K_EMPTY + ring.st]);      // the K tiles of this slot are free once dQ is done
        if (i == nv - 1) umma_commit_elect(&bars[ACC_FULL + ub]);     // written out by the last slot's worker group
        if (lane == 0) GCA_TRACE_BUF(p.prof, 6, g);
      }
      ring.next();
      if (++b == NBUF) { b = 0; bph ^= 1; }
    }
  }
}

constexpr int CW = 16;                               // key columns per pass of the worker loops

// Pass 1 for 16 keys of one query row:  P = exp2(S c - LSE),  Di += P dP,  P -> packed bf16 into
// tensor memory at `dst` (8 columns of the S region that have already been read).
__device__ __forceinline__ void pass1_cols(const uint32_t* s, const uint32_t* dp, float2 c2v, float2 nl, float2& dacc, uint32_t dst) {
  uint32_t pw[CW / 2];
#pragma unroll
  for (int q = 0; q < CW; q += 2) {
    float2 a = __ffma2_rn(f2(s[q], s[q + 1]), c2v, nl);
    a.x = ex2_approx(a.x); a.y = ex2_approx(a.y);
    dacc = __ffma2_rn(a, f2(dp[q], dp[q + 1]), dacc);
    pw[q / 2] = pack_bf16x2(a.x, a.y);
  }
  tmem_st_32x32b_x8(dst, pw);
}
// Pass 2 for the same 16 keys:  dS = P (w dP - w Di)  -> packed bf16 at `dst` (8 columns of the dP
// region that have already been read).  pk: the 8 packed words of P.
__device__ __forceinline__ void pass2_cols(const uint32_t* pk, const uint32_t* dp, float2 wv, float2 nwd, uint32_t dst) {
  uint32_t ds[CW / 2];
#pragma unroll
  for (int q = 0; q < CW; q += 2) {
    const float2 pf = f2(pk[q / 2] << 16, pk[q / 2] & 0xffff0000u);
    const float2 e = __fmul2_rn(pf, __ffma2_rn(f2(dp[q], dp[q + 1]), wv, nwd));
    ds[q / 2] = pack_bf16x2(e.x, e.y);
  }
  tmem_st_32x32b_x8(dst, ds);
}
constexpr int OUT_COLS = 16, OUT_PASSES = 64 / OUT_COLS;

__device__ void q_worker(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int wg,
                         int quad, int lane, uint32_t tmem_base) {
  // TMEM lane of this thread = 32 quad + lane = (head tile, query row) as the 64-row MMAs lay them out
  const int tile = lane >> 4;
  const int row = quad * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const bool elected = quad == 0 && lane == 0;
  const int tid = quad * 32 + lane;                             // 0..127 inside the worker group
  PairCursor c;
  c.init(p.HP);
  uint32_t ucnt = 0, g = 0;
  uint32_t b = 0, bph = 0;
  bool ok = true;
  int next_idx = q_load_row(p, c.u, c.outer, lane);
  float next_w = (c.u < p.units && lane < p.K) ? p.weights[(long long)c.outer * p.K + lane] : 0.f;
  const float2 c2v = make_float2(p.c2, p.c2);
  for (; c.u < p.units && ok; c.advance()) {
    const int my_idx = next_idx;
    const float my_w = next_w;
    {
      const int nzj = c.next_outer();
      next_idx = q_load_row(p, c.u + gridDim.x, nzj, lane);
      next_w = (c.u + gridDim.x < p.units && lane < p.K) ? p.weights[(long long)nzj * p.K + lane] : 0.f;
    }
    const unsigned mask = q_valid(p, my_idx);
    const QInfo t = q_info(p, c.inner);
    const int h = t.h0 + tile;
    const bool live = (tile == 0 || t.two) && h < p.Hq;
    const int n = c.outer / p.J, j = c.outer - n * p.J;
    __nv_bfloat16* dq_row = p.dq + n * p.dqs[0] + j * p.dqs[1] + h * p.dqs[2] + row * p.dqs[3];
    float* dwp = p.dw_part + ((long long)c.outer * p.Hq + t.h0) * p.K * 4;     // [tile][k][quarter]
    if (wg == 0) {
      // padding slots (and whole units without valid slots): zero dw partials, zero dQ rows
      const unsigned full = (p.K >= 32) ? 0xffffffffu : ((1u << p.K) - 1u);
      if (mask != full)
        for (int i = tid; i < 8 * p.K; i += 128) {
          const int tl = i / (4 * p.K), k = (i - tl * 4 * p.K) >> 2;
          if (!((mask >> k) & 1) && t.h0 + tl < p.Hq) dwp[i] = 0.f;
        }
      if (mask == 0 && live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) reinterpret_cast<uint4*>(dq_row)[cc] = z;
      }
    }
    if (mask == 0) continue;
    const uint32_t un = ucnt++;
    const long long row_off = ((long long)c.outer * p.Hq + (live ? h : t.h0)) * p.K * 64 + row;
    const float* lse_base = p.lse + row_off;
    uint4* rt_base = p.rowterm + row_off;
    for (unsigned m = mask; m; m &= m - 1, ++g) {
      const uint32_t bb = b, pp = bph;
      if (++b == NBUF) { b = 0; bph ^= 1; }
      if ((int)(g % NWG) != wg) continue;
      const int k = __ffs(m) - 1;
      const float w = __shfl_sync(0xffffffffu, my_w, k);
      const float lse = lse_base[k * 64];
      ok = mbar_wait_bounded(&bars[SP_FULL + bb], pp, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      if (elected) GCA_TRACE_BUF(p.prof, 7, g);
      tc_fence_after();
      const uint32_t tb = tlane + bb * BUF_COLS;
      // Pass 1 over the row's 64 keys, 16 at a time (ONE small loop body: after its first pass it
      // is in the instruction cache):  P = exp2(S c - LSE),  Di += P dP,  P -> packed bf16 over S
      // columns that earlier passes have already read.
      const float2 nl = make_float2(-lse, -lse);
      float2 dacc = make_float2(0.f, 0.f);
#pragma unroll 1
      for (int cpos = 0; cpos < 64; cpos += CW) {
        uint32_t s[CW], dp[CW];
        tmem_ld_32x32b_x16(tb + cpos, s);
        tmem_ld_32x32b_x16(tb + COL_DPT + cpos, dp);
        tmem_ld_wait();
        pass1_cols(s, dp, c2v, nl, dacc, tb + cpos / 2);
      }
      const float di = dacc.x + dacc.y;
      tmem_st_wait();
      if (elected) GCA_TRACE_BUF(p.prof, 8, g);
      // Pass 2:  dS = P (w dP - w Di)  -> packed bf16 over the dP columns already read.  (Issuing the
      // tensor-memory read of the next 16 columns before computing the current ones was measured
      // slower, 0.603 against 0.562 ms; so was writing dS into two regions of its own, which frees
      // the score buffer before the dQ product has run: 0.602 against 0.558 ms.)
      const float2 wv = make_float2(w, w), nwd = make_float2(-w * di, -w * di);
#pragma unroll 1
      for (int cpos = 0; cpos < 64; cpos += CW) {
        uint32_t pk[CW / 2], dp[CW];
        tmem_ld_32x32b_x8(tb + cpos / 2, pk);
        tmem_ld_32x32b_x16(tb + COL_DPT + cpos, dp);
        tmem_ld_wait();
        pass2_cols(pk, dp, wv, nwd, tb + COL_DPT + cpos / 2);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[PDS_FULL + bb]);
      if (elected) GCA_TRACE_BUF(p.prof, 9, g);
      if (live) rt_base[k * 64] = row_terms((log2_abs_clamped(w) - lse) * p.inv_c2, -di);
      // dw: sum of Di over the 16 rows this warp holds of each head's tile -> one partial per
      // (head, 16-row quarter)
      float dsum = di;
#pragma unroll
      for (int of = 8; of > 0; of >>= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, of);
      if ((lane & 15) == 0 && live) dwp[(tile * p.K + k) * 4 + quad] = dsum;
    }
    if (!ok) break;
  }
}

// The dQ writer: a warpgroup of its own, so that no worker group is held up by a unit's output (a
// worker group is tied to every NBUF-th slot; while it waited for the unit's last dQ product and
// stored the tile, ~2,000-2,800 cycles, its next slot and with it the whole ring stood still once
// per unit: 0.571 -> 0.544 ms).  Its wait is the ordinary suspending try_wait: polling with a sleep
// between probes (20 / 100 / 400 ns) was measured slower (0.584 / 0.574 / 0.558 ms).  Thread = TMEM
// lane = (head tile, query row) as in the workers.
__device__ void q_writer(const BwdQParams& p, uint64_t* bars, volatile int* abort_flag, int quad, int lane, uint32_t tmem_base) {
  const int tile = lane >> 4;
  const int row = quad * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const bool elected = quad == 0 && lane == 0;
  PairCursor c;
  c.init(p.HP);
  uint32_t ucnt = 0;
  bool ok = true;
  int next_idx = q_load_row(p, c.u, c.outer, lane);
  for (; c.u < p.units && ok; c.advance()) {
    const int my_idx = next_idx;
    next_idx = q_load_row(p, c.u + gridDim.x, c.next_outer(), lane);
    if (q_valid(p, my_idx) == 0) continue;           // the workers zero-fill units without valid slots
    const uint32_t un = ucnt++;
    const uint32_t ub = un & 1;
    const QInfo t = q_info(p, c.inner);
    const int h = t.h0 + tile;
    const bool live = (tile == 0 || t.two) && h < p.Hq;
    const int n = c.outer / p.J, j = c.outer - n * p.J;
    __nv_bfloat16* dq_row = p.dq + n * p.dqs[0] + j * p.dqs[1] + h * p.dqs[2] + row * p.dqs[3];
    ok = mbar_wait_bounded(&bars[ACC_FULL + ub], (un >> 1) & 1, abort_flag);
    if (!__all_sync(0xffffffffu, ok)) break;
    if (elected) GCA_TRACE_BUF(p.prof, 10, un);
    tc_fence_after();
    // dQ leaves in four passes of one small loop body (16 columns: TMEM -> bf16 -> one 32-byte
    // store per row)
#pragma unroll 1
    for (int part = 0; part < OUT_PASSES; ++part) {
      uint32_t v[OUT_COLS];
      tmem_ld_32x32b_x16(tlane + COL_DQ + ub * 64 + part * OUT_COLS, v);
      tmem_ld_wait();
      if (live) store16_bf16(reinterpret_cast<uint8_t*>(dq_row) + part * OUT_COLS * 2, v, p.sm_scale, p.wide_store);
    }
    tc_fence_before();
    mbar_arrive(&bars[ACC_EMPTY + ub]);
    if (elected) GCA_TRACE_BUF(p.prof, 11, un);
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
bwd_q_tc_kernel(const __grid_constant__ BwdQParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[QDO_FULL + i], 1);
      mbar_init(&bars[QDO_EMPTY + i], 2);                  // S issuers + dP issuers
      mbar_init(&bars[ACC_FULL + i], 1);
      mbar_init(&bars[ACC_EMPTY + i], 128);
    }
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(&bars[SP_FULL + i], 2);                    // S commits + dP commits
      mbar_init(&bars[PDS_FULL + i], 128);
      mbar_init(&bars[BUF_FREE + i], 1);
    }
    for (int i = 0; i < NKS; ++i) { mbar_init(&bars[K_FULL + i], 1); mbar_init(&bars[K_EMPTY + i], 1); }
    for (int i = 0; i < NVS; ++i) { mbar_init(&bars[V_FULL + i], 1); mbar_init(&bars[V_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == ISSUE_S) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == PROD_WARP && lane == 0) {
    tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_do); tma_prefetch_desc(&p.tm_k2); tma_prefetch_desc(&p.tm_v2);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 4 * NWG) q_worker(p, smem, bars, abort_flag, warp >> 2, warp & 3, lane, tmem_base);
  else if (warp == PROD_WARP) q_producer(p, smem, bars, abort_flag, lane);
  else if (warp >= WRITER_WARP) q_writer(p, bars, abort_flag, warp & 3, lane, tmem_base);
  else if (warp == ISSUE_S) q_issuer<0>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DP) q_issuer<1>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DQ) q_issuer<2>(p, smem, bars, abort_flag, lane, tmem_base);
  tc_fence_before();
  __syncthreads();
  if (warp == ISSUE_S) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

// every 64-element bf16 row of the tensor starts on a 32-byte boundary
bool rows_32b_aligned(const void* base, const int64_t* stride) {
  if (reinterpret_cast<uintptr_t>(base) & 31u) return false;
  for (int i = 0; i < 4; ++i)
    if (stride[i] % 16 != 0) return false;
  return true;
}

}  // namespace

// dw_part: (N*J, Hq, K, 4) float32 partials; rowterm: (N*J, Hq, K, 64) x 16 bytes (see BwdQParams).
int launch_bwd_q_tc(const GcaBwdArgs& a, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream) {
  const float c2 = a.sm_scale * GCA_LOG2E;
  int rc;
  auto qmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hq, a.J, a.N, st[3], st[2], st[1], st[0], box);
  };
  auto kmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hkv, a.C, a.N, st[2], st[3], st[1], st[0], box);
  };
  BwdQParams p;
  if ((rc = qmap(&p.tm_q, a.q, a.q_stride, 2)) || (rc = qmap(&p.tm_do, a.dout, a.do_stride, 2)) ||
      (rc = kmap(&p.tm_k2, a.k_cache, a.k_stride, 2)) || (rc = kmap(&p.tm_v2, a.v_cache, a.v_stride, 2)) ||
      (rc = kmap(&p.tm_k1, a.k_cache, a.k_stride, 1)) || (rc = kmap(&p.tm_v1, a.v_cache, a.v_stride, 1)))
    return rc;
  p.indices = a.indices; p.weights = a.weights; p.lse = a.lse;
  p.dq = (__nv_bfloat16*)a.dq; p.dw_part = dw_part; p.rowterm = rowterm; p.inv_c2 = 1.0f / c2; p.status = a.status;
  p.prof = profile_buffer();
  for (int i = 0; i < 4; ++i) p.dqs[i] = a.dq_stride[i];
  p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
  p.HP = (a.Hq + 1) / 2;
  const long long units = (long long)a.N * a.J * p.HP;
  if (units >= (1ll << 31) - 65536) return GCA_ERR_TOO_LARGE;
  p.units = (int)units;
  p.c2 = c2; p.sm_scale = a.sm_scale;
  p.wide_store = rows_32b_aligned(a.dq, a.dq_stride);
  if (p.units == 0) return 0;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
  bwd_q_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  GCA_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace gca
