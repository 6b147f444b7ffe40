// GCA backward, kv-major pass (dK, dV) on tcgen05 / TMEM / TMA, bf16, S = L = D = 64.
//
// Unit = (sequence n, cache chunk c, PAIR of kv heads).  K_c and V_c stay in shared memory; the
// kernel walks the inverse retrieval index (every (query chunk j, slot k) that retrieved chunk c,
// times the q heads of the group) and accumulates   dV_c += (w P)^T dO   and   dK_c += dS^T Q   in
// tensor memory across all of them; the scatter-add of the reference's gather backward
// (index_put_(accumulate=True) over the gathered gradient, model/DRT.py:198-199) becomes one tile
// store per chunk.  No atomics: the result is bit-reproducible.
//
// The scores are computed TRANSPOSED:   S^T = K_c Q^T   and   dP^T = V_c dO^T   (A = the resident
// K_c / V_c tile, B = the Q / dO tile, both K-major), so a worker thread owns one KEY row of the
// (key x query) tiles.  With   -LSE[q]   and   -Di[q] = -rowsum(P * dP)[q]   of every query row
// already in memory (the q-major pass, which runs first, writes both), the thread needs no
// reduction at all:
//     (w P)^T[key, q] = w exp2(S^T c - LSE[q]),     dS^T[key, q] = (w P)^T (dP^T - Di[q]).
// Both are written as packed bf16 into TENSOR memory, over the columns the scores came from, and
// are the A operands of the two gradient products from there (A in tensor memory has lane = row
// of A = key, exactly what the thread holds).  Shared memory, whose 128 bytes per clock bound
// these 64-wide tiles, sees neither a store nor an operand read of P^T / dS^T, and holds a deeper
// Q / dO ring instead of staging buffers.
//
// S^T and dP^T are computed per head with 64-row MMAs: a 64-row accumulator occupies lanes 0-15
// of every 32-lane quarter of tensor memory, so head B's tile, written at lane offset 16, shares
// head A's 64 columns.  Lane l of the 128 therefore holds (head (l >> 4) & 1, key 16 (l >> 5) +
// (l & 15)); the stacked 128-row gradient products inherit that row order (the accumulators dK,
// dV have it too, and the epilogue stores each lane's row where it belongs).  Two S^T / dP^T
// buffers (128 columns each) + dK + dV (128 each) fill the 512 columns.
//
// CTA = 12 warps: two worker warpgroups taking alternate iterations, one TMA producer (Q, dO,
// the (-LSE, -Di) rows and the retrieval weight of every iteration; K, V per unit), three MMA
// issuers (S^T, dP^T, gradient products).  Every wait is bounded (GCA_STATUS_TIMEOUT on expiry).
#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace gca {

namespace {

using namespace sm100;

constexpr int TILE_BYTES = 64 * 64 * 2;
constexpr int PAIR_BYTES = 2 * TILE_BYTES;
constexpr uint32_t PAIR16 = PAIR_BYTES >> 4, TILE16 = TILE_BYTES >> 4;
constexpr int NTHREADS = 384;
constexpr int PROD_WARP = 8, ISSUE_S = 9, ISSUE_DP = 10;   // warp 11: gradient-product issuer
constexpr int TMEM_COLS = 512;
constexpr uint32_t LANE16 = 16u << 16;            // TMEM lane offset of head B's 64-row tile
constexpr uint32_t IDESC_64 = umma_idesc_bf16(64, 64, 0, 0);
constexpr uint32_t IDESC_GRAD = umma_idesc_bf16(128, 128, 0, 1);   // A: tensor memory, B: MN-major, both heads' tiles
constexpr int STEP_K = 2;      // K-major operand: +32 bytes (>> 4) per K step of 16
constexpr int STEP_MN = 128;   // MN-major operand: +2048 bytes (>> 4) per K step of 16

constexpr int NQ = 4, NKV = 2;
constexpr int ROW_BYTES = 64 * 8;                            // one (head, slot): 64 x (-lse, -di)
constexpr int OFF_KV = 0;                                    // [NKV][K pair | V pair]
constexpr int OFF_QDO = OFF_KV + NKV * 2 * PAIR_BYTES;       // [NQ][Q pair | dO pair]
constexpr int OFF_NLD = OFF_QDO + NQ * 2 * PAIR_BYTES;       // [NQ][head A row | head B row]
constexpr int OFF_W = OFF_NLD + NQ * 2 * ROW_BYTES;          // [NQ] retrieval weight of the iteration
constexpr int OFF_BAR = OFF_W + 64;
constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
enum Bar { KV_FULL = 0, KV_EMPTY = KV_FULL + NKV, QDO_FULL = KV_EMPTY + NKV, QDO_EMPTY = QDO_FULL + NQ,
           SP_FULL = QDO_EMPTY + NQ, PDS_FULL = SP_FULL + 2, BUF_FREE = PDS_FULL + 2, ACC_FULL = BUF_FREE + 2,
           ACC_EMPTY = ACC_FULL + 2, NUM_BARS = ACC_EMPTY + 1 };
static_assert(NUM_BARS * 8 + 16 <= 512, "barrier block");
// Tensor-memory columns.  Buffer b (iteration g uses b = g % 2) = 128 columns: S^T at +0 and
// dP^T at +64 as float32; afterwards (w P)^T at +0 and dS^T at +64 as packed bf16 (32 columns each).
constexpr uint32_t BUF_COLS = 128, COL_DPT = 64, COL_DK = 256, COL_DV = 384;

// One bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completing on an mbarrier.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void drain(uint64_t* bars, int full0, uint32_t issued, int depth) {
  for (uint32_t back = 0; back < (uint32_t)depth && back < issued; ++back) {
    const uint32_t g = issued - 1 - back;
    for (int i = 0; i < (1 << 20); ++i)
      if (mbar_try_wait(&bars[full0 + g % depth], (g / depth) & 1)) break;
  }
}

struct BwdKvParams {
  CUtensorMap tm_q2, tm_do2, tm_q1, tm_do1, tm_k2, tm_v2;
  const float* weights;
  const float2* nld;        // (N*J, Hq, K, 64) x (-lse, -di), written by the q-major pass
  const int4* unit_tab;     // units in walking order: (first entry, one past the last, chunk id n*C + c)
  const unsigned long long* sorted_keys;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int32_t* status;
  long long dks[4], dvs[4];
  int units;
  int N, J, Hq, Hkv, G, K, C, HP;
  int wide_store;           // dk / dv rows are 32-byte aligned: 256-bit stores
  float c2, sm_scale;
};

// One lane: K + V per unit; per iteration Q + dO, the two heads' (-lse, -di) rows and the weight.
__device__ void kv_producer(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(NQ);
  uint32_t ucnt = 0, issued = 0;
  bool ok = true;
  float* sw = reinterpret_cast<float*>(smem + OFF_W);
  int4 nxt = c.u < p.units ? p.unit_tab[c.outer] : make_int4(0, 0, 0, 0);
  for (; c.u < p.units && ok; c.advance()) {
    const int beg = nxt.x, end = nxt.y, chunk = nxt.z;
    if (c.u + (int)gridDim.x < p.units) nxt = p.unit_tab[c.next_outer()];
    if (end == beg) continue;
    const uint32_t un = ucnt++;
    const int hk0 = 2 * c.inner;
    const bool two = hk0 + 1 < p.Hkv;
    const int n = chunk / p.C, ch = chunk - n * p.C;
    {
      const uint32_t kb = un % NKV;
      ok = mbar_wait_bounded(&bars[KV_EMPTY + kb], ((un / NKV) & 1) ^ 1, abort_flag);
      if (!ok) break;
      uint8_t* base = smem + OFF_KV + kb * 2 * PAIR_BYTES;
      mbar_arrive_expect_tx(&bars[KV_FULL + kb], 2 * PAIR_BYTES);
      tma_load_5d(base, &p.tm_k2, &bars[KV_FULL + kb], 0, 0, hk0, ch, n);
      tma_load_5d(base + PAIR_BYTES, &p.tm_v2, &bars[KV_FULL + kb], 0, 0, hk0, ch, n);
    }
    unsigned long long key_next = p.sorted_keys[beg];
    for (int e = beg; e < end && ok; ++e) {
      const int entry = (int)(key_next & 0xffffffffull);
      if (e + 1 < end) key_next = p.sorted_keys[e + 1];
      const int j = entry / p.K, k = entry - j * p.K;
      const long long zj = (long long)n * p.J + j;
      const float w = p.weights[zj * p.K + k];
      for (int gi = 0; gi < p.G; ++gi) {
        ok = mbar_wait_bounded(&bars[QDO_EMPTY + ring.st], ring.ph ^ 1, abort_flag);
        if (!ok) break;
        uint8_t* dst = smem + OFF_QDO + ring.st * 2 * PAIR_BYTES;
        uint8_t* nld_dst = smem + OFF_NLD + ring.st * 2 * ROW_BYTES;
        uint64_t* bar = &bars[QDO_FULL + ring.st];
        const int ha = hk0 * p.G + gi, hb = two ? (hk0 + 1) * p.G + gi : ha;
        sw[ring.st] = w;                 // ordered before the consumers' reads by the barrier's release / acquire
        mbar_arrive_expect_tx(bar, 2 * PAIR_BYTES + 2 * ROW_BYTES);
        if (p.G == 1) {
          tma_load_5d(dst, &p.tm_q2, bar, 0, 0, hk0, j, n);
          tma_load_5d(dst + PAIR_BYTES, &p.tm_do2, bar, 0, 0, hk0, j, n);
        } else {      // the two q heads of the pair are G apart: one copy per head
          tma_load_5d(dst, &p.tm_q1, bar, 0, 0, ha, j, n);
          tma_load_5d(dst + TILE_BYTES, &p.tm_q1, bar, 0, 0, hb, j, n);
          tma_load_5d(dst + PAIR_BYTES, &p.tm_do1, bar, 0, 0, ha, j, n);
          tma_load_5d(dst + PAIR_BYTES + TILE_BYTES, &p.tm_do1, bar, 0, 0, hb, j, n);
        }
        bulk_load(nld_dst, p.nld + ((zj * p.Hq + ha) * p.K + k) * 64, ROW_BYTES, bar);
        bulk_load(nld_dst + ROW_BYTES, p.nld + ((zj * p.Hq + hb) * p.K + k) * 64, ROW_BYTES, bar);
        ring.next();
        ++issued;
      }
    }
  }
  if (*abort_flag) {
    drain(bars, QDO_FULL, issued, NQ);
    drain(bars, KV_FULL, ucnt, NKV);
  }
}

// role 0: S^T per iteration;  role 1: dP^T per iteration;  role 2: dV and dK per iteration.
// All 32 lanes run this code; elect.sync inside the MMA / commit wrappers picks the issuing lane.
template <int ROLE>
__device__ void kv_issuer(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                          uint32_t tmem_base) {
  const uint64_t dKV = umma_desc_sw128(smem_u32(smem + OFF_KV));
  const uint64_t dQDO = umma_desc_sw128(smem_u32(smem + OFF_QDO));
  const uint64_t dQDOmn = umma_desc_sw128_mn_blocks(smem_u32(smem + OFF_QDO), TILE_BYTES);
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(NQ);
  uint32_t ucnt = 0, g = 0;
  bool ok = true;
  int4 nxt = c.u < p.units ? p.unit_tab[c.outer] : make_int4(0, 0, 0, 0);
  for (; c.u < p.units && ok; c.advance()) {
    const int beg = nxt.x, end = nxt.y;
    if (c.u + (int)gridDim.x < p.units) nxt = p.unit_tab[c.next_outer()];
    const int niter = (end - beg) * p.G;
    if (niter == 0) continue;
    const uint32_t un = ucnt++;
    const uint32_t kb = un % NKV;
    if (ROLE != 2) ok = mbar_wait_warp(&bars[KV_FULL + kb], (un / NKV) & 1, abort_flag, lane);
    else ok = mbar_wait_warp(&bars[ACC_EMPTY], (un & 1) ^ 1, abort_flag, lane);
    for (int i = 0; i < niter && ok; ++i, ++g) {
      const uint64_t stage = ring.st * 2 * PAIR16;
      const uint32_t b = g & 1;                           // buffer = worker group of this iteration
      const uint32_t tbuf = tmem_base + b * BUF_COLS;
      if (ROLE != 2) {
        ok = mbar_wait_warp(&bars[QDO_FULL + ring.st], ring.ph, abort_flag, lane);
        // the buffer's previous contents ((w P)^T, dS^T of iteration g - 2) have been consumed
        if (ok) ok = mbar_wait_warp(&bars[BUF_FREE + b], ((g >> 1) & 1) ^ 1, abort_flag, lane);
        if (!ok) break;
        tc_fence_after();
        const uint64_t a = dKV + kb * 2 * PAIR16 + (ROLE == 0 ? 0u : PAIR16);       // K pair | V pair
        const uint64_t bq = dQDO + stage + (ROLE == 0 ? 0u : PAIR16);               // Q pair | dO pair
        const uint32_t d = tbuf + (ROLE == 0 ? 0u : COL_DPT);
#pragma unroll
        for (int tl = 0; tl < 2; ++tl)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ss_elect(d + (tl ? LANE16 : 0u), a + tl * TILE16 + kk * STEP_K, bq + tl * TILE16 + kk * STEP_K,
                               IDESC_64, (uint32_t)(kk > 0));
        umma_commit_elect(&bars[SP_FULL + b]);            // the barrier expects both the S^T and the dP^T commit
      } else {
        ok = mbar_wait_warp(&bars[PDS_FULL + b], (g >> 1) & 1, abort_flag, lane);
        if (!ok) break;
        tc_fence_after();
        // dV += (w P)^T dO, dK += dS^T Q: A from tensor memory (lane = key row, 8 columns per
        // K step of 16 query rows), B = dO / Q read N-contiguous (MN-major) across both heads' tiles
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts_elect(tmem_base + COL_DV, tbuf + kk * 8, dQDOmn + stage + PAIR16 + kk * STEP_MN, IDESC_GRAD,
                             (uint32_t)(i > 0 || kk > 0));
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts_elect(tmem_base + COL_DK, tbuf + COL_DPT + kk * 8, dQDOmn + stage + kk * STEP_MN, IDESC_GRAD,
                             (uint32_t)(i > 0 || kk > 0));
        umma_commit_elect(&bars[BUF_FREE + b]);
        umma_commit_elect(&bars[QDO_EMPTY + ring.st]);   // Q / dO of this iteration are free once dV, dK are done
        if (i == niter - 1) umma_commit_elect(&bars[ACC_FULL + b]);   // written out by the last iteration's worker group
      }
      ring.next();
    }
  }
}

// One thread, one key row of one head: s = S^T row (64 query columns), dp = dP^T row.
// nld: the head's 64 x (-lse, -di).  Produces (w P)^T and dS^T rows, packed bf16 in query order.
__device__ __forceinline__ void row_transposed(const uint32_t* s, const uint32_t* dp, const float4* nld, float c2, float w,
                                               uint32_t* pw_out, uint32_t* ds_out) {
  const float2 c2v = make_float2(c2, c2), wv = make_float2(w, w);
#pragma unroll
  for (int q = 0; q < 64; q += 4) {
    const float4 x0 = nld[q / 2], x1 = nld[q / 2 + 1];           // (-lse, -di) of query rows q, q+1 | q+2, q+3
    float2 a0 = __ffma2_rn(f2(s[q + 0], s[q + 1]), c2v, make_float2(x0.x, x0.z));
    float2 a1 = __ffma2_rn(f2(s[q + 2], s[q + 3]), c2v, make_float2(x1.x, x1.z));
    a0.x = ex2_approx(a0.x); a0.y = ex2_approx(a0.y); a1.x = ex2_approx(a1.x); a1.y = ex2_approx(a1.y);
    const float2 p0 = __fmul2_rn(a0, wv), p1 = __fmul2_rn(a1, wv);
    const float2 e0 = __fmul2_rn(p0, __fadd2_rn(f2(dp[q + 0], dp[q + 1]), make_float2(x0.y, x0.w)));
    const float2 e1 = __fmul2_rn(p1, __fadd2_rn(f2(dp[q + 2], dp[q + 3]), make_float2(x1.y, x1.w)));
    pw_out[q / 2] = pack_bf16x2(p0.x, p0.y); pw_out[q / 2 + 1] = pack_bf16x2(p1.x, p1.y);
    ds_out[q / 2] = pack_bf16x2(e0.x, e0.y); ds_out[q / 2 + 1] = pack_bf16x2(e1.x, e1.y);
  }
}

constexpr int OUT_COLS = 16, OUT_PASSES = 64 / OUT_COLS;

__device__ void kv_worker(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int wg,
                          int quad, int lane, uint32_t tmem_base) {
  // TMEM lane of this thread = 32 quad + lane = (head tile, key row) as the 64-row MMAs lay them out
  const int tile = lane >> 4;
  const int row = quad * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const uint32_t coff = (uint32_t)tile * 64u;          // this head's columns of the stacked accumulators
  const bool elected = quad == 0 && lane == 0;
  const float* sw = reinterpret_cast<const float*>(smem + OFF_W);
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(NQ);
  uint32_t ucnt = 0, g = 0;
  bool ok = true;
  uint32_t epi = 0;                             // units this group has written out
  int4 nxt = c.u < p.units ? p.unit_tab[c.outer] : make_int4(0, 0, 0, 0);
  for (; c.u < p.units && ok; c.advance()) {
    const int beg = nxt.x, end = nxt.y, chunk = nxt.z;
    if (c.u + (int)gridDim.x < p.units) nxt = p.unit_tab[c.next_outer()];
    const int hk = 2 * c.inner + tile;
    const bool live = hk < p.Hkv;
    const int n = chunk / p.C, ch = chunk - n * p.C;
    __nv_bfloat16* dk_row = p.dk + n * p.dks[0] + ch * p.dks[1] + row * p.dks[2] + hk * p.dks[3];
    __nv_bfloat16* dv_row = p.dv + n * p.dvs[0] + ch * p.dvs[1] + row * p.dvs[2] + hk * p.dvs[3];
    if (end == beg) {                           // nobody retrieved this chunk: zero gradient
      if (wg == 0 && live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) { reinterpret_cast<uint4*>(dk_row)[cc] = z; reinterpret_cast<uint4*>(dv_row)[cc] = z; }
      }
      continue;
    }
    const uint32_t un = ucnt++;
    const uint32_t kb = un % NKV;
    const int niter = (end - beg) * p.G;
    bool my_unit = false;                     // this group ran the unit's last iteration: it writes dK, dV
    for (int i = 0; i < niter; ++i, ++g, ring.next()) {
      my_unit = (int)(g & 1) == wg;
      if (!my_unit) continue;
      const uint32_t b = g & 1;
      ok = mbar_wait_bounded(&bars[SP_FULL + b], (g >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      // S^T / dP^T of the unit's last iteration are complete: its K / V tiles are no longer needed
      if (elected && i == niter - 1) mbar_arrive(&bars[KV_EMPTY + kb]);
      tc_fence_after();
      uint32_t s[64], dp[64];
      const uint32_t tb = tlane + b * BUF_COLS;
      tmem_ld_32x32b_x32(tb, s);
      tmem_ld_32x32b_x32(tb + 32, s + 32);
      tmem_ld_32x32b_x32(tb + COL_DPT, dp);
      tmem_ld_32x32b_x32(tb + COL_DPT + 32, dp + 32);
      const float w = sw[ring.st];
      const float4* nld = reinterpret_cast<const float4*>(smem + OFF_NLD + ring.st * 2 * ROW_BYTES + tile * ROW_BYTES);
      tmem_ld_wait();
      uint32_t pw[32], ds[32];
      row_transposed(s, dp, nld, p.c2, w, pw, ds);
      tmem_st_32x32b_x32(tb, pw);
      tmem_st_32x32b_x32(tb + COL_DPT, ds);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars[PDS_FULL + b]);
    }
    if (!ok) break;
    if (my_unit) {
      ok = mbar_wait_bounded(&bars[ACC_FULL + wg], epi & 1, abort_flag);
      ++epi;
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      // The two tiles leave in eight passes of ONE small loop body (16 columns: TMEM -> bf16 ->
      // one 32-byte store per row): after the first pass the body is in the instruction cache,
      // where a straight-line conversion of all 128 columns (~250 instructions, executed once per
      // unit) runs at instruction-fetch speed.
#pragma unroll 1
      for (int part = 0; part < 2 * OUT_PASSES; ++part) {
        const bool is_dv = part >= OUT_PASSES;
        const int pp = is_dv ? part - OUT_PASSES : part;
        uint32_t v[OUT_COLS];
        tmem_ld_32x32b_x16(tlane + (is_dv ? COL_DV : COL_DK) + coff + pp * OUT_COLS, v);
        tmem_ld_wait();
        if (live)
          store16_bf16(reinterpret_cast<uint8_t*>(is_dv ? dv_row : dk_row) + pp * OUT_COLS * 2, v, is_dv ? 1.0f : p.sm_scale,
                       p.wide_store);
      }
      tc_fence_before();
      mbar_arrive(&bars[ACC_EMPTY]);
    }
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
bwd_kv_tc_kernel(const __grid_constant__ BwdKvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[SP_FULL + i], 2);                              // S^T commit + dP^T commit
      mbar_init(&bars[PDS_FULL + i], 128);
      mbar_init(&bars[BUF_FREE + i], 1);
      mbar_init(&bars[ACC_FULL + i], 1);
    }
    mbar_init(&bars[ACC_EMPTY], 128);
    for (int i = 0; i < NKV; ++i) { mbar_init(&bars[KV_FULL + i], 1); mbar_init(&bars[KV_EMPTY + i], 1); }
    for (int i = 0; i < NQ; ++i) { mbar_init(&bars[QDO_FULL + i], 1); mbar_init(&bars[QDO_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == ISSUE_S) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == PROD_WARP && lane == 0) {
    tma_prefetch_desc(&p.tm_q2); tma_prefetch_desc(&p.tm_do2); tma_prefetch_desc(&p.tm_k2); tma_prefetch_desc(&p.tm_v2);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 8) kv_worker(p, smem, bars, abort_flag, warp >> 2, warp & 3, lane, tmem_base);
  else if (warp == PROD_WARP) { if (lane == 0) kv_producer(p, smem, bars, abort_flag); }
  else if (warp == ISSUE_S) kv_issuer<0>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DP) kv_issuer<1>(p, smem, bars, abort_flag, lane, tmem_base);
  else kv_issuer<2>(p, smem, bars, abort_flag, lane, tmem_base);
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

// nld: (N*J, Hq, K, 64) x (-lse, -di) as the q-major pass wrote it into the workspace.
int launch_bwd_kv_tc(const GcaBwdArgs& a, const Csr& csr, const float2* nld, int sms, cudaStream_t stream) {
  BwdKvParams p;
  int rc;
  auto qmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hq, a.J, a.N, st[3], st[2], st[1], st[0], box);
  };
  auto kmap = [&](CUtensorMap* m, const void* base, const int64_t* st, int box) {
    return make_tile_map_5d(m, base, 64, 64, a.Hkv, a.C, a.N, st[2], st[3], st[1], st[0], box);
  };
  if ((rc = qmap(&p.tm_q2, a.q, a.q_stride, 2)) || (rc = qmap(&p.tm_do2, a.dout, a.do_stride, 2)) ||
      (rc = qmap(&p.tm_q1, a.q, a.q_stride, 1)) || (rc = qmap(&p.tm_do1, a.dout, a.do_stride, 1)) ||
      (rc = kmap(&p.tm_k2, a.k_cache, a.k_stride, 2)) || (rc = kmap(&p.tm_v2, a.v_cache, a.v_stride, 2)))
    return rc;
  p.weights = a.weights; p.nld = nld; p.unit_tab = csr.unit_tab; p.sorted_keys = csr.sorted_keys;
  p.dk = (__nv_bfloat16*)a.dk_cache; p.dv = (__nv_bfloat16*)a.dv_cache; p.status = a.status;
  for (int i = 0; i < 4; ++i) { p.dks[i] = a.dk_stride[i]; p.dvs[i] = a.dv_stride[i]; }
  p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
  p.HP = (a.Hkv + 1) / 2;
  const long long units = (long long)a.N * a.C * p.HP;
  if (units >= (1ll << 31) - 65536) return GCA_ERR_TOO_LARGE;
  p.units = (int)units;
  p.c2 = a.sm_scale * GCA_LOG2E; p.sm_scale = a.sm_scale;
  p.wide_store = rows_32b_aligned(a.dk_cache, a.dk_stride) && rows_32b_aligned(a.dv_cache, a.dv_stride);
  if (p.units == 0) return 0;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_kv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
  bwd_kv_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  GCA_CUDA_CHECK(cudaGetLastError());
  return 0;
}

}  // namespace gca
