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
// (key x query) tiles.  What the backward needs per QUERY row -- the log-sum-exp, the retrieval
// weight and Di = rowsum(P * dP) -- is known before this kernel starts (the q-major pass, which
// runs first, writes it), and it enters through the TENSOR CORE: every S^T / dP^T product gets a
// fifth K step whose A operand is a constant tile of ones and whose B operand holds, per query
// row, three bf16 values that sum to (log2|w| - LSE) / c for S^T and to -Di for dP^T (three bf16
// = 24 mantissa bits; the products with 1.0 are exact and accumulate in float32).  The
// accumulators then hold   S^T + (log2|w| - LSE) / c   and   dP^T - Di,   and a thread computes
//     |w| P^T = exp2(c * acc_S),        |w| dS^T = |w| P^T * acc_dP
// with no per-column operand at all: no shared-memory loads (which take hundreds of cycles while
// the MMAs saturate shared memory), no reduction, six instructions per pair of elements.  The
// sign of w is applied by the gradient MMAs (negate-A bit of the instruction descriptor).
// Both results are written as packed bf16 into TENSOR memory, over the columns the scores came
// from, and are the A operands of the two gradient products from there (A in tensor memory has
// lane = row of A = key, exactly what the thread holds).  Shared memory, whose 128 bytes per
// clock bound these 64-wide tiles, sees neither a store nor an operand read of P^T / dS^T.
//
// Every product is computed per head with 64-row MMAs: a 64-row operand or accumulator occupies
// lanes 0-15 of every 32-lane quarter of tensor memory, so head B's tiles, placed at lane offset
// 16, share head A's columns.  Lane l of the 128 therefore holds (head (l >> 4) & 1, key
// 16 (l >> 5) + (l & 15)) in the score buffers, in the packed A operands and in the accumulators
// alike.  A score buffer (S^T | dP^T, 128 columns) is free again only when the gradient products
// that read it have completed, and a buffer goes through MMA -> workers -> MMA -> release in
// ~3,000 cycles, so the number of buffers sets the iteration rate: with 64-column accumulators
// (dK, dV: 128 columns for both heads) THREE buffers fit in the 512 columns.
//
// CTA: NBUF * SPLIT worker warpgroups (the SPLIT groups of a buffer share its columns and take
// every NBUF-th iteration), one TMA producer (Q, dO and the per-row term tiles of every
// iteration; K, V per unit) and the MMA issuers (S^T, dP^T, dV, dK).  Every wait is bounded
// (GCA_STATUS_TIMEOUT on expiry).
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
// Worker arrangement: NBUF score buffers, SPLIT worker warpgroups per buffer, each taking
// 64 / SPLIT of the query columns of every key row of its buffer's iterations.
#ifndef GCA_KV_NBUF
#define GCA_KV_NBUF 3
#endif
#ifndef GCA_KV_SPLIT
#define GCA_KV_SPLIT 1
#endif
#ifndef GCA_KV_GRAD2
#define GCA_KV_GRAD2 1
#endif
constexpr int NBUF = GCA_KV_NBUF, SPLIT = GCA_KV_SPLIT, NG = NBUF * SPLIT;
constexpr int GRAD_ISSUERS = GCA_KV_GRAD2 ? 2 : 1;       // dV and dK from one warp, or from a warp each
static_assert(NBUF == 2 || NBUF == 3, "score buffers");
// One issuing warp per product (two for the gradients with GRAD2).  Measured slower: one issuing
// warp per HEAD (0.955 against 0.615 ms: both heads of an iteration share the buffer's columns, and
// every extra polling warp loads the shared-memory path); a warpgroup of its own that writes dK /
// dV so that no worker group is held up by a unit's output (0.668 ms, 0.70-0.81 with sleeping
// waits: with single accumulators the gradient issuers wait for the writer either way, and four
// more resident warps cost more than the freed worker group gains).
// Probing the next iteration's barriers before the current iteration's MMAs are issued (a 7 % gain in the
// q-major kernel) was measured slower here: 0.634 against 0.613 ms.
#ifndef GCA_KV_PREPROBE
#define GCA_KV_PREPROBE 0
#endif
constexpr int PROD_WARP = 4 * NG, ISSUE_S = PROD_WARP + 1, ISSUE_DP = ISSUE_S + 1, ISSUE_DV = ISSUE_DP + 1;       // dK issuer (GRAD2): ISSUE_DV + 1
constexpr int NTHREADS = (ISSUE_DV + GRAD_ISSUERS) * 32;
constexpr int WCOLS = 64 / SPLIT;                        // query columns of a key row that one group handles
constexpr int TMEM_COLS = 512;
constexpr uint32_t LANE16 = 16u << 16;            // TMEM lane offset of head B's 64-row tile
constexpr uint32_t IDESC_64 = umma_idesc_bf16(64, 64, 0, 0);
constexpr uint32_t IDESC_GRAD = umma_idesc_bf16(64, 64, 0, 1);     // A: tensor memory, B: MN-major
constexpr uint32_t IDESC_NEG_A = 1u << 13;                         // negate the A operand
constexpr int STEP_K = 2;      // K-major operand: +32 bytes (>> 4) per K step of 16
constexpr int STEP_MN = 128;   // MN-major operand: +2048 bytes (>> 4) per K step of 16

constexpr int NQ = 4, NKV = 2;
// Row-term tile of one (head, slot): 64 query rows x 16 bytes (eight bf16: a0 a1 a2 b0 b1 b2 0 0),
// which is the first 8-element column block of a K-major operand without swizzle (8-row groups
// 128 bytes apart); the second column block of the K step of 16 is a block of zeros.
constexpr int RT_BYTES = 64 * 16;
constexpr int OFF_KV = 0;                                    // [NKV][K pair | V pair]
constexpr int OFF_QDO = OFF_KV + NKV * 2 * PAIR_BYTES;       // [NQ][Q pair | dO pair]
constexpr int OFF_RT = OFF_QDO + NQ * 2 * PAIR_BYTES;        // [NQ][head A tile | head B tile]
constexpr int OFF_ONES_S = OFF_RT + NQ * 2 * RT_BYTES;       // 64 rows x (1 1 1 0 0 0 0 0): picks a0 + a1 + a2
constexpr int OFF_ONES_DP = OFF_ONES_S + RT_BYTES;           // 64 rows x (0 0 0 1 1 1 0 0): picks b0 + b1 + b2
constexpr int OFF_ZERO = OFF_ONES_DP + RT_BYTES;             // 64 rows x 16 bytes of zeros
constexpr int OFF_W = OFF_ZERO + RT_BYTES;                   // [NQ] retrieval weight of the iteration (its sign is used)
constexpr int OFF_BAR = OFF_W + 64;
constexpr int SMEM_BYTES = OFF_BAR + 512 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
enum Bar { KV_FULL = 0, KV_EMPTY = KV_FULL + NKV, QDO_FULL = KV_EMPTY + NKV, QDO_EMPTY = QDO_FULL + NQ,
           SP_FULL = QDO_EMPTY + NQ, PDS_FULL = SP_FULL + NBUF, BUF_FREE = PDS_FULL + NBUF, ACC_FULL = BUF_FREE + NBUF,
           ACC_EMPTY = ACC_FULL + NBUF, NUM_BARS = ACC_EMPTY + 1 };
static_assert(NUM_BARS * 8 + 16 <= 512, "barrier block");
// Tensor-memory columns.  Buffer b (iteration g uses b = g % NBUF) = 128 columns: S^T at +0 and
// dP^T at +64 as float32; afterwards |w| P^T at +0 and |w| dS^T at +64 as packed bf16 (32 columns
// each, see packed_col).  Behind the buffers dK and dV, 64 columns each.
constexpr uint32_t BUF_COLS = 128, COL_DPT = 64, COL_DK = NBUF * BUF_COLS, COL_DV = COL_DK + 64;
static_assert(COL_DV + 64 <= TMEM_COLS, "tensor memory");

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
  const uint4* rowterm;     // (N*J, Hq, K) tiles of 64 x 16 bytes, written by the q-major pass
  const int4* unit_tab;     // units in walking order: (first entry, one past the last, chunk id n*C + c)
  const unsigned long long* sorted_keys;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int32_t* status;
  long long* prof;          // event trace of block 0 (profile builds only), or nullptr
  long long dks[4], dvs[4];
  int units;
  int N, J, Hq, Hkv, G, K, C, HP;
  int wide_store;           // dk / dv rows are 32-byte aligned: 256-bit stores
  float c2, sm_scale;
};

// One lane: K + V per unit; per iteration Q + dO, the two heads' row-term tiles and the weight.
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
        uint8_t* rt_dst = smem + OFF_RT + ring.st * 2 * RT_BYTES;
        uint64_t* bar = &bars[QDO_FULL + ring.st];
        const int ha = hk0 * p.G + gi, hb = two ? (hk0 + 1) * p.G + gi : ha;
        GCA_TRACE_BUF(p.prof, 0, issued);
        sw[ring.st] = w;                 // ordered before the consumers' reads by the barrier's release / acquire
        mbar_arrive_expect_tx(bar, 2 * PAIR_BYTES + 2 * RT_BYTES);
        if (p.G == 1) {
          tma_load_5d(dst, &p.tm_q2, bar, 0, 0, hk0, j, n);
          tma_load_5d(dst + PAIR_BYTES, &p.tm_do2, bar, 0, 0, hk0, j, n);
        } else {      // the two q heads of the pair are G apart: one copy per head
          tma_load_5d(dst, &p.tm_q1, bar, 0, 0, ha, j, n);
          tma_load_5d(dst + TILE_BYTES, &p.tm_q1, bar, 0, 0, hb, j, n);
          tma_load_5d(dst + PAIR_BYTES, &p.tm_do1, bar, 0, 0, ha, j, n);
          tma_load_5d(dst + PAIR_BYTES + TILE_BYTES, &p.tm_do1, bar, 0, 0, hb, j, n);
        }
        bulk_load(rt_dst, p.rowterm + ((zj * p.Hq + ha) * p.K + k) * 64, RT_BYTES, bar);
        bulk_load(rt_dst + RT_BYTES, p.rowterm + ((zj * p.Hq + hb) * p.K + k) * 64, RT_BYTES, bar);
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

// (w P)^T / dS^T of query columns 16 kk .. 16 kk + 15 (one K step of the gradient products): the
// group that handled those columns wrote them, packed, at the start of its own column range.
__host__ __device__ constexpr uint32_t packed_col(int kk) {
  return (uint32_t)((16 * kk) / WCOLS * WCOLS + ((16 * kk) % WCOLS) / 2);
}

// role 0: S^T per iteration;  role 1: dP^T per iteration;  role 2: dV (and dK when there is one
// gradient issuer);  role 3: dK.  All 32 lanes run this code; elect.sync inside the MMA / commit
// wrappers picks the issuing lane.
template <int ROLE>
__device__ void kv_issuer(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                          uint32_t tmem_base) {
  const uint64_t dKV = umma_desc_sw128(smem_u32(smem + OFF_KV));
  const uint64_t dQDO = umma_desc_sw128(smem_u32(smem + OFF_QDO));
  const uint64_t dQDOmn = umma_desc_sw128_mn_blocks(smem_u32(smem + OFF_QDO), TILE_BYTES);
  const uint32_t zero_addr = smem_u32(smem + OFF_ZERO);
  const uint32_t ones_addr = smem_u32(smem + (ROLE == 0 ? OFF_ONES_S : OFF_ONES_DP));
  const uint64_t dOnes = umma_desc_nosw_k(ones_addr, zero_addr - ones_addr, 128);
  const float* sw = reinterpret_cast<const float*>(smem + OFF_W);
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(NQ);
  uint32_t ucnt = 0, g = 0;
  uint32_t b = 0, bph = 0;                                // g % NBUF and the parity of g / NBUF
  bool ok = true;
  int4 nxt = c.u < p.units ? p.unit_tab[c.outer] : make_int4(0, 0, 0, 0);
  for (; c.u < p.units && ok; c.advance()) {
    const int beg = nxt.x, end = nxt.y;
    if (c.u + (int)gridDim.x < p.units) nxt = p.unit_tab[c.next_outer()];
    const int niter = (end - beg) * p.G;
    if (niter == 0) continue;
    const uint32_t un = ucnt++;
    const uint32_t kb = un % NKV;
    if (ROLE < 2) ok = mbar_wait_warp(&bars[KV_FULL + kb], (un / NKV) & 1, abort_flag, lane);
    else ok = mbar_wait_warp(&bars[ACC_EMPTY], (un & 1) ^ 1, abort_flag, lane);
    bool pre_a = false, pre_b = false;           // early probe results for the coming iteration
    for (int i = 0; i < niter && ok; ++i, ++g) {
      const uint64_t stage = ring.st * 2 * PAIR16;
      const uint32_t tbuf = tmem_base + b * BUF_COLS;
      if (ROLE < 2) {
        // the tiles have landed AND the buffer's previous contents (the packed A operands of iteration
        // g - NBUF) have been consumed: both barriers are probed at once (one shared-memory round trip)
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 1, g);
        // (probed while the previous iteration's MMAs were being issued, when there was one in this unit)
        ok = mbar_wait_warp2_probed(&bars[QDO_FULL + ring.st], ring.ph, pre_a, &bars[BUF_FREE + b], bph ^ 1, pre_b, abort_flag);
        if (!ok) break;
        if (lane == 0 && ROLE == 0) GCA_TRACE_BUF(p.prof, 2, g);
        tc_fence_after();
        pre_a = pre_b = false;
        if (GCA_KV_PREPROBE && i + 1 < niter) {          // the next iteration's two barriers: their shared-memory round
          const uint32_t nst = ring.st + 1 == (uint32_t)ring.depth ? 0u : ring.st + 1, nph = nst ? ring.ph : ring.ph ^ 1;   // trip runs under the MMA issue
          const uint32_t nb = b + 1 == NBUF ? 0u : b + 1, nbph = nb ? bph : bph ^ 1;
          pre_a = mbar_test_wait(&bars[QDO_FULL + nst], nph);
          pre_b = mbar_test_wait(&bars[BUF_FREE + nb], nbph ^ 1);
        }
        const uint64_t a = dKV + kb * 2 * PAIR16 + (ROLE == 0 ? 0u : PAIR16);       // K pair | V pair
        const uint64_t bq = dQDO + stage + (ROLE == 0 ? 0u : PAIR16);               // Q pair | dO pair
        const uint32_t d = tbuf + (ROLE == 0 ? 0u : COL_DPT);
        // fifth K step: A = the constant ones tile, B = the head's row-term tile of this stage
        const uint32_t rt = smem_u32(smem + OFF_RT + ring.st * 2 * RT_BYTES);
#pragma unroll
        for (int tl = 0; tl < 2; ++tl) {
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_bf16_ss_elect(d + (tl ? LANE16 : 0u), a + tl * TILE16 + kk * STEP_K, bq + tl * TILE16 + kk * STEP_K,
                               IDESC_64, (uint32_t)(kk > 0));
          umma_bf16_ss_elect(d + (tl ? LANE16 : 0u), dOnes, umma_desc_nosw_k(rt + tl * RT_BYTES, zero_addr - (rt + tl * RT_BYTES), 128),
                             IDESC_64, 1u);
        }
        umma_commit_elect(&bars[SP_FULL + b]);            // the barrier expects both the S^T and the dP^T commit
        if (lane == 0) GCA_TRACE_BUF(p.prof, 3 + ROLE, g);
      } else {
        ok = mbar_wait_warp2_probed(&bars[PDS_FULL + b], bph, pre_a, &bars[PDS_FULL + b], bph, true, abort_flag);
        if (!ok) break;
        if (lane == 0 && ROLE == 2) GCA_TRACE_BUF(p.prof, 5, g);
        tc_fence_after();
        pre_a = false;
        if (GCA_KV_PREPROBE && i + 1 < niter) {
          const uint32_t nb = b + 1 == NBUF ? 0u : b + 1, nbph = nb ? bph : bph ^ 1;
          pre_a = mbar_test_wait(&bars[PDS_FULL + nb], nbph);
        }
        // the workers produced |w| P^T and |w| dS^T: a negative weight negates both A operands
        const uint32_t idesc = IDESC_GRAD | (sw[ring.st] < 0.f ? IDESC_NEG_A : 0u);
        // dV += (w P)^T dO, dK += dS^T Q, per head: A from tensor memory (lane = key row, 8 columns
        // per K step of 16 query rows), B = the head's dO / Q tile read N-contiguous (MN-major)
        if (ROLE == 2) {
#pragma unroll
          for (int tl = 0; tl < 2; ++tl) {
  #pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_bf16_ts_elect(tmem_base + COL_DV + (tl ? LANE16 : 0u), tbuf + (tl ? LANE16 : 0u) + packed_col(kk),
                                 dQDOmn + stage + PAIR16 + tl * TILE16 + kk * STEP_MN, idesc, (uint32_t)(i > 0 || kk > 0));
          }
        }
        if (ROLE == 3 || GRAD_ISSUERS == 1) {
#pragma unroll
          for (int tl = 0; tl < 2; ++tl) {
  #pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_bf16_ts_elect(tmem_base + COL_DK + (tl ? LANE16 : 0u), tbuf + COL_DPT + (tl ? LANE16 : 0u) + packed_col(kk),
                                 dQDOmn + stage + tl * TILE16 + kk * STEP_MN, idesc, (uint32_t)(i > 0 || kk > 0));
          }
        }
        umma_commit_elect(&bars[BUF_FREE + b]);
        umma_commit_elect(&bars[QDO_EMPTY + ring.st]);   // Q / dO of this iteration are free once dV, dK are done
        if (i == niter - 1) umma_commit_elect(&bars[ACC_FULL + b]);   // written out by the last iteration's worker groups
        if (lane == 0 && ROLE == 2) GCA_TRACE_BUF(p.prof, 6, g);
      }
      ring.next();
      if (++b == NBUF) { b = 0; bph ^= 1; }
    }
  }
}

// One thread, one key row of one head, CW query columns: s = the S^T accumulator values (scores +
// (log2|w| - lse) / c), dp = the dP^T accumulator values (dP - Di).  Produces |w| P^T and |w| dS^T,
// packed bf16 in query order (CW / 2 words each).
#ifndef GCA_KV_CW
#define GCA_KV_CW 16
#endif
constexpr int CW = GCA_KV_CW < WCOLS ? GCA_KV_CW : WCOLS;      // query columns per pass of the worker loop
__device__ __forceinline__ void cols_transposed(const uint32_t* s, const uint32_t* dp, float2 c2v, uint32_t* pw_out,
                                                uint32_t* ds_out) {
#pragma unroll
  for (int q = 0; q < CW; q += 2) {
    float2 a = __fmul2_rn(f2(s[q], s[q + 1]), c2v);
    a.x = ex2_approx(a.x); a.y = ex2_approx(a.y);
    const float2 e = __fmul2_rn(a, f2(dp[q], dp[q + 1]));
    pw_out[q / 2] = pack_bf16x2(a.x, a.y);
    ds_out[q / 2] = pack_bf16x2(e.x, e.y);
  }
}

__device__ __forceinline__ void tmem_ld_cw(uint32_t taddr, uint32_t* r) {
  if (CW == 32) tmem_ld_32x32b_x32(taddr, r); else if (CW == 16) tmem_ld_32x32b_x16(taddr, r); else tmem_ld_32x32b_x8(taddr, r);
}
__device__ __forceinline__ void tmem_st_half(uint32_t taddr, const uint32_t* r) {
  if (CW == 32) tmem_st_32x32b_x16(taddr, r); else if (CW == 16) tmem_st_32x32b_x8(taddr, r); else tmem_st_32x32b_x4(taddr, r);
}

constexpr int OUT_COLS = 16, OUT_PASSES = 64 / OUT_COLS;

__device__ void kv_worker(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int wg,
                          int quad, int lane, uint32_t tmem_base) {
  // TMEM lane of this thread = 32 quad + lane = (head tile, key row) as the 64-row MMAs lay them out
  const int tile = lane >> 4;
  const int row = quad * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const bool elected = quad == 0 && lane == 0;
  PairCursor c;
  c.init(p.HP);
  Ring ring; ring.init(NQ);
  uint32_t ucnt = 0, g = 0;
  bool ok = true;
  uint32_t epi = 0;                             // units this group has helped to write out
  uint32_t b = 0, bph = 0;                      // g % NBUF and the parity of g / NBUF
  const int my_buf = wg / SPLIT, part = wg % SPLIT;
  int4 nxt = c.u < p.units ? p.unit_tab[c.outer] : make_int4(0, 0, 0, 0);
  for (; c.u < p.units && ok; c.advance()) {
    const int beg = nxt.x, end = nxt.y, chunk = nxt.z;
    if (c.u + (int)gridDim.x < p.units) nxt = p.unit_tab[c.next_outer()];
    if (end == beg) {                           // nobody retrieved this chunk: zero gradient
      const int hk = 2 * c.inner + tile;
      if (wg == 0 && hk < p.Hkv) {
        const int n = chunk / p.C, ch = chunk - n * p.C;
        __nv_bfloat16* dk_row = p.dk + n * p.dks[0] + ch * p.dks[1] + row * p.dks[2] + hk * p.dks[3];
        __nv_bfloat16* dv_row = p.dv + n * p.dvs[0] + ch * p.dvs[1] + row * p.dvs[2] + hk * p.dvs[3];
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) { reinterpret_cast<uint4*>(dk_row)[cc] = z; reinterpret_cast<uint4*>(dv_row)[cc] = z; }
      }
      continue;
    }
    const uint32_t un = ucnt++;
    const uint32_t kb = un % NKV;
    const int niter = (end - beg) * p.G;
    bool my_unit = false;                     // this group took part in the unit's last iteration: it helps write dK, dV
    for (int i = 0; i < niter; ++i, ++g, ring.next()) {
      const uint32_t bb = b, pp = bph;
      if (++b == NBUF) { b = 0; bph ^= 1; }
      my_unit = (int)bb == my_buf;
      if (!my_unit) continue;
      ok = mbar_wait_bounded(&bars[SP_FULL + bb], pp, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 7, g);
      // S^T / dP^T of the unit's last iteration are complete: its K / V tiles are no longer needed
      if (elected && part == 0 && i == niter - 1) mbar_arrive(&bars[KV_EMPTY + kb]);
      tc_fence_after();
      const uint32_t tb = tlane + bb * BUF_COLS + part * WCOLS;
      const float2 c2v = make_float2(p.c2, p.c2);
      // The group's columns are processed in passes of CW columns by ONE small loop body (tensor
      // memory -> registers -> exp2, product -> packed bf16 -> tensor memory).  A straight-line
      // treatment of all the columns, executed once per iteration, runs at instruction-fetch speed;
      // a small body is in the instruction cache after its first pass (measured: 64 columns
      // straight-line 2,140 cycles per row, four passes of 16 columns 1,780; issuing the
      // tensor-memory read of a pass before the previous pass is computed made the body larger
      // and the kernel 25 % slower).  The packed results of pass i land on columns that this
      // group's passes <= i have already read.
#pragma unroll 1
      for (int cpos = 0; cpos < WCOLS; cpos += CW) {
        uint32_t s[CW], dp[CW], pw[CW / 2], ds[CW / 2];
        tmem_ld_cw(tb + cpos, s);
        tmem_ld_cw(tb + COL_DPT + cpos, dp);
        tmem_ld_wait();
        if (elected && part == 0 && cpos == 0) GCA_TRACE_BUF(p.prof, 8, g);
        cols_transposed(s, dp, c2v, pw, ds);
        tmem_st_half(tb + cpos / 2, pw);
        tmem_st_half(tb + COL_DPT + cpos / 2, ds);
        if (elected && part == 0 && cpos == 0) GCA_TRACE_BUF(p.prof, 13, g);
      }
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 14, g);
      tmem_st_wait();
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 15, g);
      tc_fence_before();
      mbar_arrive(&bars[PDS_FULL + bb]);
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 9, g);
    }
    if (!ok) break;
    if (my_unit) {
      ok = mbar_wait_bounded(&bars[ACC_FULL + my_buf], epi & 1, abort_flag);
      ++epi;
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 10, un);
      tc_fence_after();
      const int hk = 2 * c.inner + tile;
      const bool live = hk < p.Hkv;
      const int n = chunk / p.C, ch = chunk - n * p.C;
      __nv_bfloat16* dk_row = p.dk + n * p.dks[0] + ch * p.dks[1] + row * p.dks[2] + hk * p.dks[3];
      __nv_bfloat16* dv_row = p.dv + n * p.dvs[0] + ch * p.dvs[1] + row * p.dvs[2] + hk * p.dvs[3];
      // The two tiles leave in eight passes of ONE small loop body (16 columns: TMEM -> bf16 ->
      // one 32-byte store per row), shared out among the groups of the unit's last iteration: after
      // its first pass a group finds the body in the instruction cache, where a straight-line
      // conversion of all 128 columns (~250 instructions, executed once per unit) runs at
      // instruction-fetch speed.
#pragma unroll 1
      for (int pass = part; pass < 2 * OUT_PASSES; pass += SPLIT) {
        const bool is_dv = pass >= OUT_PASSES;
        const int pq = is_dv ? pass - OUT_PASSES : pass;
        uint32_t v[OUT_COLS];
        tmem_ld_32x32b_x16(tlane + (is_dv ? COL_DV : COL_DK) + pq * OUT_COLS, v);
        tmem_ld_wait();
        if (live)
          store16_bf16(reinterpret_cast<uint8_t*>(is_dv ? dv_row : dk_row) + pq * OUT_COLS * 2, v, is_dv ? 1.0f : p.sm_scale,
                       p.wide_store);
      }
      tc_fence_before();
      mbar_arrive(&bars[ACC_EMPTY]);
      if (elected && part == 0) GCA_TRACE_BUF(p.prof, 11, un);
      if (elected && part == 0 && p.prof != nullptr && blockIdx.x == 0 && un < 256u) p.prof[64 + 12 * 256 + un] = g;
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
    for (int i = 0; i < NBUF; ++i) {
      mbar_init(&bars[SP_FULL + i], 2);                              // S^T commit + dP^T commit
      mbar_init(&bars[PDS_FULL + i], 128 * SPLIT);
      mbar_init(&bars[BUF_FREE + i], GRAD_ISSUERS);             // one commit per gradient issuer
      mbar_init(&bars[ACC_FULL + i], GRAD_ISSUERS);
    }
    mbar_init(&bars[ACC_EMPTY], 128 * SPLIT);
    for (int i = 0; i < NKV; ++i) { mbar_init(&bars[KV_FULL + i], 1); mbar_init(&bars[KV_EMPTY + i], 1); }
    for (int i = 0; i < NQ; ++i) { mbar_init(&bars[QDO_FULL + i], 1); mbar_init(&bars[QDO_EMPTY + i], GRAD_ISSUERS); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x < 64) {          // the constant operand tiles of the fifth K step (one 16-byte row per thread)
    const uint32_t one2 = 0x3f803f80u, one_lo = 0x00003f80u, one_hi = 0x3f800000u;     // bf16 1.0
    reinterpret_cast<uint4*>(smem + OFF_ONES_S)[threadIdx.x] = make_uint4(one2, one_lo, 0u, 0u);     // 1 1 1 0 0 0 0 0
    reinterpret_cast<uint4*>(smem + OFF_ONES_DP)[threadIdx.x] = make_uint4(0u, one_hi, one2, 0u);    // 0 0 0 1 1 1 0 0
    reinterpret_cast<uint4*>(smem + OFF_ZERO)[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();      // written through the generic proxy, read by the MMAs through the async proxy
  }
  if (warp == ISSUE_S) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == PROD_WARP && lane == 0) {
    tma_prefetch_desc(&p.tm_q2); tma_prefetch_desc(&p.tm_do2); tma_prefetch_desc(&p.tm_k2); tma_prefetch_desc(&p.tm_v2);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 4 * NG) kv_worker(p, smem, bars, abort_flag, warp >> 2, warp & 3, lane, tmem_base);
  else if (warp == PROD_WARP) { if (lane == 0) kv_producer(p, smem, bars, abort_flag); }
  else if (warp == ISSUE_S) kv_issuer<0>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DP) kv_issuer<1>(p, smem, bars, abort_flag, lane, tmem_base);
  else if (warp == ISSUE_DV) kv_issuer<2>(p, smem, bars, abort_flag, lane, tmem_base);
  else kv_issuer<3>(p, smem, bars, abort_flag, lane, tmem_base);
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

// rowterm: the per-row term tiles as the q-major pass wrote them into the workspace (1 KB per
// (row block, head, slot)).
int launch_bwd_kv_tc(const GcaBwdArgs& a, const Csr& csr, const uint4* rowterm, int sms, cudaStream_t stream) {
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
  p.weights = a.weights; p.rowterm = rowterm; p.unit_tab = csr.unit_tab; p.sorted_keys = csr.sorted_keys;
  p.dk = (__nv_bfloat16*)a.dk_cache; p.dv = (__nv_bfloat16*)a.dv_cache; p.status = a.status;
  p.prof = profile_buffer();
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
