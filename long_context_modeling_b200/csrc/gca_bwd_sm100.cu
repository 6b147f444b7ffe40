// GCA backward, q-major pass (dQ, dw and the per-row terms the kv-major pass needs) on tcgen05 /
// TMEM / TMA, bf16, S = L = D = 64, plus the launch sequence of the whole tensor-core backward.
//
// Unit = (sequence n, query chunk j, PAIR of q heads) as in the forward.  Per retrieved slot the
// kernel recomputes  S = Q K^T  and  dP = dO V^T;  one thread per query row forms
// P = exp2(S c - LSE),  Di = rowsum(P * dP)  (which replaces the reference's extra o = v^T p^T
// product, ltriton/gca.py:382),  dS = w P (dP - Di);  dQ += dS K_k accumulates over the K slots in
// tensor memory, and the per-head parts of  dw_k = sum_rows Di  go to a partials buffer that a tiny
// fixed-order kernel reduces.  For every (row, slot) the two per-row terms of the kv-major pass,
// (log2|w| - LSE) / c and -Di, are also written to the workspace, each split into three bf16
// values: the kv-major pass (gca_bwd_kv_sm100.cu), which runs AFTER this one, adds them to its
// recomputed scores with one extra MMA K step and then needs neither a row reduction nor any
// per-row operand of its own (the reference hands Di from one of its two kernels to the other in
// the same way, ltriton/gca.py:385,459).
//
// The two heads of a pair are stacked so that every tcgen05.mma is a 128-row instruction whose
// diagonal 64x64 blocks are the two heads' results (the issue cost of an MMA does not depend on
// its shape, so fewer, larger instructions win).  dS stays in TENSOR memory (bf16, two keys per
// 32-bit column, written by the thread that computed the row) and is the A operand of the dQ
// product from there: shared memory, whose 128 bytes per clock bound these 64-wide tiles, sees
// neither its store nor its operand reads.  K as the N-contiguous B operand of that product is
// read through an MN-major descriptor spanning both heads' tiles: nothing is transposed in software.
// Output tiles leave in rolled passes of 16 columns (one small loop body that stays in the
// instruction cache) rather than as ~150 straight-line instructions executed once per unit.
//
// CTA = 12 warps: two worker warpgroups (thread = TMEM lane = row) taking alternate slots, one
// TMA producer, and THREE MMA issuers: S, dP and dQ each have their own warp, because S and dP
// share one TMEM buffer each and their issue latency sits on the critical path of every slot.
// Neither pass uses atomics, so gradients are bit-reproducible.  Every wait is bounded
// (GCA_STATUS_TIMEOUT on expiry).
#include <cstdlib>

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
constexpr uint32_t PAIR16 = PAIR_BYTES >> 4;
constexpr int NTHREADS = 384;
constexpr int PROD_WARP = 8, ISSUE_S = 9, ISSUE_DP = 10;   // warp 11: dQ issuer
constexpr int TMEM_COLS = 512;
// S and dP are single stacked 128-row tiles (per-head 64-row products were measured 5 % slower
// here: twice the S / dP instructions, and the slots are bound by the K ring, not by the S / dP
// turnaround).
constexpr uint32_t QCOL_S = 0, QCOL_DP = 128;

// Four K steps of one stacked product.  a_step / b_step: descriptor advance per K step of 16.
// Called by ALL lanes of the issuing warp (converged, warp-uniform operands); elect.sync picks
// the lane that issues: ~100 cycles per instruction instead of ~150 inside an `if (lane == 0)`.
constexpr int STEP_K = 2;      // K-major operand: +32 bytes (>> 4)
constexpr int STEP_MN = 128;   // MN-major operand: +2048 bytes (>> 4)
__device__ __forceinline__ void mma4(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, int a_step, int b_step,
                                     bool accumulate_first) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) umma_bf16_ss_elect(d, a + kk * a_step, b + kk * b_step, idesc, (uint32_t)(accumulate_first || kk > 0));
}

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

// One thread, one query row.  s: raw scores (overwritten by P), dp: raw dP.  dS stays in registers,
// packed two keys per word in key order (the layout of an A operand in tensor memory).  ds may
// alias s.  Returns Di = rowsum(P * dP).
__device__ __forceinline__ float row_backward_packed(uint32_t* s, const uint32_t* dp, float lse, float c2, float w,
                                                     uint32_t* ds) {
  const float2 c2v = make_float2(c2, c2), nl = make_float2(-lse, -lse);
  float2 d0 = make_float2(0.f, 0.f), d1 = d0, d2 = d0, d3 = d0;
#pragma unroll
  for (int c = 0; c < 64; c += 8) {
    float2 a0 = __ffma2_rn(f2(s[c + 0], s[c + 1]), c2v, nl), a1 = __ffma2_rn(f2(s[c + 2], s[c + 3]), c2v, nl);
    float2 a2 = __ffma2_rn(f2(s[c + 4], s[c + 5]), c2v, nl), a3 = __ffma2_rn(f2(s[c + 6], s[c + 7]), c2v, nl);
    a0.x = ex2_approx(a0.x); a0.y = ex2_approx(a0.y); a1.x = ex2_approx(a1.x); a1.y = ex2_approx(a1.y);
    a2.x = ex2_approx(a2.x); a2.y = ex2_approx(a2.y); a3.x = ex2_approx(a3.x); a3.y = ex2_approx(a3.y);
    d0 = __ffma2_rn(a0, f2(dp[c + 0], dp[c + 1]), d0); d1 = __ffma2_rn(a1, f2(dp[c + 2], dp[c + 3]), d1);
    d2 = __ffma2_rn(a2, f2(dp[c + 4], dp[c + 5]), d2); d3 = __ffma2_rn(a3, f2(dp[c + 6], dp[c + 7]), d3);
    s[c + 0] = __float_as_uint(a0.x); s[c + 1] = __float_as_uint(a0.y); s[c + 2] = __float_as_uint(a1.x); s[c + 3] = __float_as_uint(a1.y);
    s[c + 4] = __float_as_uint(a2.x); s[c + 5] = __float_as_uint(a2.y); s[c + 6] = __float_as_uint(a3.x); s[c + 7] = __float_as_uint(a3.y);
  }
  const float2 dsum = __fadd2_rn(__fadd2_rn(d0, d1), __fadd2_rn(d2, d3));
  const float di = dsum.x + dsum.y;
  const float2 wv = make_float2(w, w), ndi = make_float2(-di, -di);
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    const float2 p0 = __fmul2_rn(f2(s[8 * c8 + 0], s[8 * c8 + 1]), wv), p1 = __fmul2_rn(f2(s[8 * c8 + 2], s[8 * c8 + 3]), wv);
    const float2 p2 = __fmul2_rn(f2(s[8 * c8 + 4], s[8 * c8 + 5]), wv), p3 = __fmul2_rn(f2(s[8 * c8 + 6], s[8 * c8 + 7]), wv);
    const float2 e0 = __fmul2_rn(p0, __fadd2_rn(f2(dp[8 * c8 + 0], dp[8 * c8 + 1]), ndi));
    const float2 e1 = __fmul2_rn(p1, __fadd2_rn(f2(dp[8 * c8 + 2], dp[8 * c8 + 3]), ndi));
    const float2 e2 = __fmul2_rn(p2, __fadd2_rn(f2(dp[8 * c8 + 4], dp[8 * c8 + 5]), ndi));
    const float2 e3 = __fmul2_rn(p3, __fadd2_rn(f2(dp[8 * c8 + 6], dp[8 * c8 + 7]), ndi));
    ds[4 * c8 + 0] = pack_bf16x2(e0.x, e0.y); ds[4 * c8 + 1] = pack_bf16x2(e1.x, e1.y);
    ds[4 * c8 + 2] = pack_bf16x2(e2.x, e2.y); ds[4 * c8 + 3] = pack_bf16x2(e3.x, e3.y);
  }
  return di;
}

__device__ __forceinline__ void drain(uint64_t* bars, int full0, uint32_t issued, int depth) {
  for (uint32_t back = 0; back < (uint32_t)depth && back < issued; ++back) {
    const uint32_t g = issued - 1 - back;
    for (int i = 0; i < (1 << 20); ++i)
      if (mbar_try_wait(&bars[full0 + g % depth], (g / depth) & 1)) break;
  }
}

// Output tiles leave in OUT_PASSES passes of OUT_COLS columns per row (see the epilogues).
#ifndef GCA_OUT_COLS
#define GCA_OUT_COLS 16
#endif
constexpr int OUT_COLS = GCA_OUT_COLS, OUT_PASSES = 64 / OUT_COLS;
__device__ __forceinline__ void out_pass_load(uint32_t taddr, uint32_t* v) {
  if (OUT_COLS == 32) tmem_ld_32x32b_x32(taddr, v); else tmem_ld_32x32b_x16(taddr, v);
  tmem_ld_wait();
}
__device__ __forceinline__ void out_pass_store(uint8_t* dst, const uint32_t* v, float scale, bool wide) {
  store16_bf16(dst, v, scale, wide);
  if (OUT_COLS == 32) store16_bf16(dst + 32, v + 16, scale, wide);
}

// =============================================================================================
// q-major kernel: dQ, dw
// =============================================================================================
namespace qk {
// dS never touches shared memory: the worker that computed a row writes it (bf16, two keys per
// 32-bit column) into tensor memory, where the dQ product reads it as its A operand.  The 32 KB
// this frees hold one more K and one more V stage.
constexpr int NKS = 5, NVS = 4;
constexpr int OFF_QDO = 0;                                   // [2 bufs][Q pair | dO pair]
constexpr int OFF_K = OFF_QDO + 2 * 2 * PAIR_BYTES;          // [NKS][K pair]
constexpr int OFF_V = OFF_K + NKS * PAIR_BYTES;              // [NVS][V pair]
constexpr int OFF_BAR = OFF_V + NVS * PAIR_BYTES;
constexpr int OFF_IDX = OFF_BAR + 512;
constexpr int SMEM_BYTES = OFF_IDX + 256 + 1024;
enum Bar { QDO_FULL = 0, QDO_EMPTY = 2, K_FULL = 4, K_EMPTY = K_FULL + NKS, V_FULL = K_EMPTY + NKS,
           V_EMPTY = V_FULL + NVS, SP_FULL = V_EMPTY + NVS, SP_EMPTY = SP_FULL + 2, DS_FULL = SP_EMPTY + 1,
           DS_EMPTY = DS_FULL + 2, DQ_FULL = DS_EMPTY + 2, DQ_EMPTY = DQ_FULL + 2, NUM_BARS = DQ_EMPTY + 1 };
// TMEM columns: S | dP | dQ (one accumulator: the group that wrote the unit's last dS copies it
// to registers and releases it before it stores) | dS of even slots | dS of odd slots
constexpr uint32_t QCOL_DQ = 256, QCOL_DS = 384, DS_COLS = 32;
}  // namespace qk

struct BwdQParams {
  CUtensorMap tm_q, tm_do, tm_k2, tm_v2, tm_k1, tm_v1;
  const int32_t* indices;
  const float* weights;
  const float* lse;
  __nv_bfloat16* dq;
  float* dw_part;           // (N*J, Hq, K, 2): two half-tile partials per (row block, head, slot)
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
  using namespace qk;
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

// role 0: S per slot;  role 1: dP per slot;  role 2: dQ += dS K per slot
template <int ROLE>
__device__ void q_issuer(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                         uint32_t tmem_base) {
  using namespace qk;
  const uint64_t dQDO = umma_desc_sw128(smem_u32(smem + OFF_QDO));
  const uint64_t dK = umma_desc_sw128(smem_u32(smem + OFF_K)), dV = umma_desc_sw128(smem_u32(smem + OFF_V));
  const uint64_t dKmn = umma_desc_sw128_mn_blocks(smem_u32(smem + OFF_K), TILE_BYTES);
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(ROLE == 1 ? NVS : NKS);
  uint32_t ucnt = 0, g = 0;
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
    const int ncol = t.share ? 64 : 128;
    if (ROLE != 2) ok = mbar_wait_warp(&bars[QDO_FULL + ub], uph, abort_flag, lane);
    else ok = mbar_wait_warp(&bars[DQ_EMPTY], (un & 1) ^ 1, abort_flag, lane);
    for (int i = 0; i < nv && ok; ++i, ++g) {
      if (ROLE != 2) {
        ok = mbar_wait_warp(&bars[(ROLE == 0 ? K_FULL : V_FULL) + ring.st], ring.ph, abort_flag, lane);
        if (ok) ok = mbar_wait_warp(&bars[SP_EMPTY], (g & 1) ^ 1, abort_flag, lane);
        if (!ok) break;
        tc_fence_after();
        const uint32_t idesc = umma_idesc_bf16(128, ncol, 0, 0);
        const uint64_t q = dQDO + ub * 2 * PAIR16;
        if (ROLE == 0) mma4(tmem_base + QCOL_S, q, dK + ring.st * PAIR16, idesc, STEP_K, STEP_K, false);
        else mma4(tmem_base + QCOL_DP, q + PAIR16, dV + ring.st * PAIR16, idesc, STEP_K, STEP_K, false);
        umma_commit_elect(&bars[SP_FULL + (g & 1)]);    // the barrier expects both the S and the dP commit
      } else {
        const uint32_t sb = g & 1;
        ok = mbar_wait_warp(&bars[DS_FULL + sb], (g >> 1) & 1, abort_flag, lane);
        if (!ok) break;
        tc_fence_after();
        // dQ += dS K_k : A = dS (tensor memory), B = K_k (MN-major, both heads' tiles)
        const uint32_t idesc = umma_idesc_bf16(128, ncol, 0, 1);
        const uint64_t b = dKmn + ring.st * PAIR16;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts_elect(tmem_base + QCOL_DQ, tmem_base + QCOL_DS + sb * DS_COLS + kk * 8, b + kk * STEP_MN, idesc,
                             (uint32_t)(i > 0 || kk > 0));
        umma_commit_elect(&bars[DS_EMPTY + sb]);
        umma_commit_elect(&bars[K_EMPTY + ring.st]);     // the K tiles of this slot are free once dQ is done
        // dQ is written out by the worker group of the unit's last slot (it has just finished
        // and its next slot is two slots away)
        if (i == nv - 1) umma_commit_elect(&bars[DQ_FULL + sb]);
      }
      ring.next();
    }
  }
}

__device__ void q_worker(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int wg,
                         int quad, int lane, uint32_t tmem_base) {
  using namespace qk;
  const int tile = quad >> 1;
  const int row = (quad & 1) * 32 + lane;
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const bool elected = quad == 0 && lane == 0;
  const int tid = quad * 32 + lane;                             // 0..127 inside the worker group
  PairCursor c;
  c.init(p.HP);
  uint32_t ucnt = 0, g = 0;
  bool ok = true;
  uint32_t epi = 0;                             // units this group has written out
  PhaseTimer pf;
  pf.init(false);
  int next_idx = q_load_row(p, c.u, c.outer, lane);
  float next_w = (c.u < p.units && lane < p.K) ? p.weights[(long long)c.outer * p.K + lane] : 0.f;
  for (; c.u < p.units && ok; c.advance()) {
    pf.lap(8);
    const int my_idx = next_idx;
    const float my_w = next_w;
    {
      const int nzj = c.next_outer();
      next_idx = q_load_row(p, c.u + gridDim.x, nzj, lane);
      next_w = (c.u + gridDim.x < p.units && lane < p.K) ? p.weights[(long long)nzj * p.K + lane] : 0.f;
    }
    const unsigned mask = q_valid(p, my_idx);
    pf.lap(9);
    const QInfo t = q_info(p, c.inner);
    const int h = t.h0 + tile;
    const bool live = (tile == 0 || t.two) && h < p.Hq;
    const uint32_t coff = t.share ? 0u : (uint32_t)tile * 64u;
    const int n = c.outer / p.J, j = c.outer - n * p.J;
    __nv_bfloat16* dq_row = p.dq + n * p.dqs[0] + j * p.dqs[1] + h * p.dqs[2] + row * p.dqs[3];
    float* dwp = p.dw_part + ((long long)c.outer * p.Hq + t.h0) * p.K * 2;     // [tile][k][half]
    if (wg == 0) {
      // padding slots (and whole units without valid slots): zero dw partials, zero dQ rows
      const unsigned full = (p.K >= 32) ? 0xffffffffu : ((1u << p.K) - 1u);
      if (mask != full)
        for (int i = tid; i < 4 * p.K; i += 128) {
          const int tl = i / (2 * p.K), k = (i - tl * 2 * p.K) >> 1;
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
    const uint32_t ub = un & 1;
    const long long row_off = ((long long)c.outer * p.Hq + (live ? h : t.h0)) * p.K * 64 + row;
    const float* lse_base = p.lse + row_off;
    uint4* rt_base = p.rowterm + row_off;
    pf.lap(10);
    bool my_unit = false;                       // this group owns the unit's last slot: it writes dQ
    for (unsigned m = mask; m; m &= m - 1, ++g) {
      my_unit = (int)(g & 1) == wg;
      if (!my_unit) continue;
      pf.lap(11);
      const int k = __ffs(m) - 1;
      const bool last = (m & (m - 1)) == 0;
      const float w = __shfl_sync(0xffffffffu, my_w, k);
      const float lse = lse_base[k * 64];
      const uint32_t sb = g & 1;
      pf.lap(7);
      ok = mbar_wait_bounded(&bars[SP_FULL + sb], (g >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      pf.lap(0);
      if (elected) {                         // S/dP done: the V stage (and at the end Q/dO) can be refilled
        mbar_arrive(&bars[V_EMPTY + g % NVS]);
        if (last) mbar_arrive(&bars[QDO_EMPTY + ub]);
      }
      tc_fence_after();
      uint32_t s[64], dp[64];
      tmem_ld_32x32b_x32(tlane + QCOL_S + coff, s);
      tmem_ld_32x32b_x32(tlane + QCOL_S + coff + 32, s + 32);
      tmem_ld_32x32b_x32(tlane + QCOL_DP + coff, dp);
      tmem_ld_32x32b_x32(tlane + QCOL_DP + coff + 32, dp + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars[SP_EMPTY]);
      pf.lap(1);
      ok = mbar_wait_bounded(&bars[DS_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      pf.lap(2);
      float di = row_backward_packed(s, dp, lse, p.c2, w, s);
      if (live) rt_base[k * 64] = row_terms((log2_abs_clamped(w) - lse) * p.inv_c2, -di);
      tmem_st_32x32b_x32(tlane + QCOL_DS + sb * DS_COLS, s);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[DS_FULL + sb]);
      pf.lap(3);
      // dw: sum of Di over the 32 rows this warp holds of its tile -> one partial per warp
#pragma unroll
      for (int of = 16; of > 0; of >>= 1) di += __shfl_xor_sync(0xffffffffu, di, of);
      if (lane == 0 && live) dwp[(tile * p.K + k) * 2 + (quad & 1)] = di;
      pf.lap(4);
    }
    if (!ok) break;
    if (my_unit) {
      pf.lap(7);
      ok = mbar_wait_bounded(&bars[DQ_FULL + wg], epi & 1, abort_flag);
      ++epi;
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      pf.lap(5);
      tc_fence_after();
      // dQ leaves in four passes of one small loop body (16 columns: TMEM -> bf16 -> one 32-byte
      // store per row): after the first pass the body is in the instruction cache
#pragma unroll 1
      for (int part = 0; part < OUT_PASSES; ++part) {
        uint32_t v[OUT_COLS];
        out_pass_load(tlane + QCOL_DQ + coff + part * OUT_COLS, v);
        if (live) out_pass_store(reinterpret_cast<uint8_t*>(dq_row) + part * OUT_COLS * 2, v, p.sm_scale, p.wide_store);
      }
      tc_fence_before();
      mbar_arrive(&bars[DQ_EMPTY]);
      pf.lap(6);
    }
  }
  pf.lap(7);
  pf.dump(p.prof + 36);
}

__global__ void __launch_bounds__(NTHREADS, 1)
bwd_q_tc_kernel(const __grid_constant__ BwdQParams p) {
  using namespace qk;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[QDO_FULL + i], 1); mbar_init(&bars[QDO_EMPTY + i], 1);
      mbar_init(&bars[SP_FULL + i], 2);                              // S commit + dP commit
      mbar_init(&bars[DS_FULL + i], 128); mbar_init(&bars[DS_EMPTY + i], 1);
      mbar_init(&bars[DQ_FULL + i], 1);
    }
    mbar_init(&bars[DQ_EMPTY], 128);
    mbar_init(&bars[SP_EMPTY], 128);
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
  if (warp < 8) q_worker(p, smem, bars, abort_flag, warp >> 2, warp & 3, lane, tmem_base);
  else if (warp == PROD_WARP) q_producer(p, smem, bars, abort_flag, lane);
  else if (warp == ISSUE_S) q_issuer<0>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DP) q_issuer<1>(p, smem, bars, abort_flag, lane, tmem_base);
  else q_issuer<2>(p, smem, bars, abort_flag, lane, tmem_base);
  tc_fence_before();
  __syncthreads();
  if (warp == ISSUE_S) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

}  // namespace

bool bwd_tc_available() { return true; }

// every 64-element bf16 row of the tensor starts on a 32-byte boundary
static bool rows_32b_aligned(const void* base, const int64_t* stride) {
  if (reinterpret_cast<uintptr_t>(base) & 31u) return false;
  for (int i = 0; i < 4; ++i)
    if (stride[i] % 16 != 0) return false;
  return true;
}

int launch_bwd_kv_tc(const GcaBwdArgs& a, const Csr& csr, const uint4* rowterm, int sms, cudaStream_t stream);
int launch_bwd_q_tc(const GcaBwdArgs& a, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream);

#ifdef GCA_Q_STACKED
int bwd_tc_dw_parts() { return 2; }
#else
int bwd_tc_dw_parts() { return 4; }
#endif

// Stage order inside one call: the q-major pass first (it writes the per-row terms), then the
// kv-major pass, which reads them.  A caller that runs the stages in separate calls must keep
// that order on the stream (or synchronise between them).
int launch_bwd_tc(const GcaBwdArgs& a, const Csr& csr, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream, unsigned stages) {
  if (a.dtype != GCA_BF16 || a.S != 64 || a.L != 64 || a.D != 64 || a.K > 32) return GCA_ERR_ALGO;
  const float c2 = a.sm_scale * GCA_LOG2E;
  int rc;
  auto qmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hq, a.J, a.N, st[3], st[2], st[1], st[0], box);
  };
  auto kmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hkv, a.C, a.N, st[2], st[3], st[1], st[0], box);
  };
#ifndef GCA_Q_STACKED
  if (stages & GCA_BWD_STAGE_Q) {
    if ((rc = launch_bwd_q_tc(a, dw_part, rowterm, sms, stream))) return rc;
  }
#else
  if (stages & GCA_BWD_STAGE_Q) {
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
    if (p.units > 0) {
      GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, qk::SMEM_BYTES));
      const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
      bwd_q_tc_kernel<<<grid, NTHREADS, qk::SMEM_BYTES, stream>>>(p);
      GCA_CUDA_CHECK(cudaGetLastError());
    }
  }
#endif
  if (stages & GCA_BWD_STAGE_KV) {
    if ((rc = launch_bwd_kv_tc(a, csr, rowterm, sms, stream))) return rc;
  }
  return 0;
}

}  // namespace gca
