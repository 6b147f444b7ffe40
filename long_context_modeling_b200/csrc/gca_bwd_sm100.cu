// GCA backward on tcgen05 / TMEM / TMA, bf16, S = L = D = 64.  Two persistent kernels,
// neither uses atomics, so gradients are bit-reproducible:
//
//  * bwd_kv_tc_kernel  (kv-major)  unit = (sequence n, cache chunk c, PAIR of kv heads).
//    K_c and V_c stay in shared memory; the kernel walks the inverse retrieval index (every
//    (query chunk j, slot k) that retrieved chunk c, times the q heads of the group) and
//    accumulates   dV_c += (w P)^T dO   and   dK_c += dS^T Q   in TMEM across all of them;
//    the scatter-add of the reference's gather backward becomes one tile store per chunk.
//  * bwd_q_tc_kernel   (q-major)   unit = (n, query chunk j, PAIR of q heads) as in the
//    forward: dQ += dS K_k accumulated over the K slots in TMEM, and the per-head part of
//    dw_k = sum_rows <dO, O_k> = sum_rows rowsum(P * dP).
//
// Per (query tile, key tile) both kernels recompute  S = Q K^T  and  dP = dO V^T  with two
// 64x64x64 MMAs, then one thread per query row forms  P = exp2(S c - LSE),
// Di = rowsum(P*dP),  dS = w P (dP - Di)  and stages bf16 tiles for the follow-up MMAs.
// Transposed operands (P^T, dS^T, and dO / Q / K as the N-contiguous B operand) are read
// through MN-major shared-memory descriptors, so nothing is transposed in software.
// As in the forward, two 64-row tiles are interleaved in the TMEM lanes (lanes 0-15 /
// 16-31 of every quarter) so all 128 worker threads own a full row.
#include <cstdlib>

#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace gca {

namespace {

using namespace sm100;

constexpr int TILE_BYTES = 64 * 64 * 2;
constexpr int NSTAGE = 3;
constexpr int NTHREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr uint32_t LANE16 = 16u << 16;

constexpr uint32_t IDESC_KK = umma_idesc_bf16(64, 64, 0, 0);   // A K-major, B K-major   (S, dP)
constexpr uint32_t IDESC_KM = umma_idesc_bf16(64, 64, 0, 1);   // A K-major, B MN-major  (dQ)
constexpr uint32_t IDESC_MM = umma_idesc_bf16(64, 64, 1, 1);   // A MN-major, B MN-major (dV, dK)

__device__ __forceinline__ void named_barrier_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// four K steps of one 64x64x64 product
__device__ __forceinline__ void mma_tile(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, int a_step, int b_step,
                                         bool accumulate_first) {
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(d, a + kk * a_step, b + kk * b_step, idesc, (accumulate_first || kk > 0));
}
constexpr int STEP_K = 2;      // K-major operand: +32 bytes per K step (>> 4)
constexpr int STEP_MN = 128;   // MN-major operand: +2048 bytes per K step (>> 4)

// One thread, one query row: P, Di, dS from the S and dP rows.  Writes (w P) and/or dS as
// bf16 into swizzled K-major tiles.  Returns Di (unweighted).
__device__ __forceinline__ float row_backward(const uint32_t* s, const uint32_t* dp, float lse, float c2, float w,
                                              uint8_t* pw_row, uint8_t* ds_row, int row) {
  float p[64];
  float di = 0.f;
#pragma unroll
  for (int c = 0; c < 64; ++c) {
    p[c] = ex2_approx(fmaf(__uint_as_float(s[c]), c2, -lse));
    di = fmaf(p[c], __uint_as_float(dp[c]), di);
  }
  const int sw = row & 7;
  if (pw_row) {
#pragma unroll
    for (int c8 = 0; c8 < 8; ++c8) {
      uint4 v;
      v.x = pack_bf16x2(p[8 * c8 + 0] * w, p[8 * c8 + 1] * w);
      v.y = pack_bf16x2(p[8 * c8 + 2] * w, p[8 * c8 + 3] * w);
      v.z = pack_bf16x2(p[8 * c8 + 4] * w, p[8 * c8 + 5] * w);
      v.w = pack_bf16x2(p[8 * c8 + 6] * w, p[8 * c8 + 7] * w);
      *reinterpret_cast<uint4*>(pw_row + ((c8 ^ sw) << 4)) = v;
    }
  }
#pragma unroll
  for (int c8 = 0; c8 < 8; ++c8) {
    float e[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = p[8 * c8 + i] * w * (__uint_as_float(dp[8 * c8 + i]) - di);
    uint4 v;
    v.x = pack_bf16x2(e[0], e[1]); v.y = pack_bf16x2(e[2], e[3]);
    v.z = pack_bf16x2(e[4], e[5]); v.w = pack_bf16x2(e[6], e[7]);
    *reinterpret_cast<uint4*>(ds_row + ((c8 ^ sw) << 4)) = v;
  }
  return di;
}

__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const uint32_t* acc, float scale) {
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    uint4 v;
    v.x = pack_bf16x2(__uint_as_float(acc[8 * c + 0]) * scale, __uint_as_float(acc[8 * c + 1]) * scale);
    v.y = pack_bf16x2(__uint_as_float(acc[8 * c + 2]) * scale, __uint_as_float(acc[8 * c + 3]) * scale);
    v.z = pack_bf16x2(__uint_as_float(acc[8 * c + 4]) * scale, __uint_as_float(acc[8 * c + 5]) * scale);
    v.w = pack_bf16x2(__uint_as_float(acc[8 * c + 6]) * scale, __uint_as_float(acc[8 * c + 7]) * scale);
    reinterpret_cast<uint4*>(dst)[c] = v;
  }
}

// =============================================================================================
// q-major kernel: dQ, dw
// =============================================================================================
namespace qk {
constexpr int OFF_QDO = 0;                                   // [2 bufs][Qa Qb dOa dOb]
constexpr int OFF_KV = OFF_QDO + 2 * 4 * TILE_BYTES;         // [NSTAGE][Ka Kb Va Vb]
constexpr int OFF_DS = OFF_KV + NSTAGE * 4 * TILE_BYTES;     // [2 bufs][dSa dSb]
constexpr int OFF_DW = OFF_DS + 2 * 2 * TILE_BYTES;          // float [2 units][32 slots][2 tiles][4 warps]
constexpr int OFF_BAR = OFF_DW + 2 * 32 * 2 * 4 * 4;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
enum Bar { QDO_FULL = 0, QDO_EMPTY = 2, KV_FULL = 4, KV_EMPTY = 4 + NSTAGE, SP_FULL = 4 + 2 * NSTAGE,
           SP_EMPTY = SP_FULL + 2, DS_FULL = SP_EMPTY + 2, DS_EMPTY = DS_FULL + 2, DQ_FULL = DS_EMPTY + 2,
           DQ_EMPTY = DQ_FULL + 2, NUM_BARS = DQ_EMPTY + 2 };
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256;
}  // namespace qk

struct BwdQParams {
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  const int32_t* indices;
  const float* weights;
  const float* lse;
  __nv_bfloat16* dq;
  float* dw_part;
  int32_t* status;
  long long dqs[4];
  long long units;
  int N, J, Hq, Hkv, G, K, C, HP;
  float c2, sm_scale;
};

struct QUnit { int zj, n, j, h0, two, hk0, hk1, share; };
__device__ __forceinline__ QUnit decode_qunit(const BwdQParams& p, long long u) {
  QUnit t;
  t.zj = (int)(u / p.HP);
  const int hp = (int)(u % p.HP);
  t.n = t.zj / p.J; t.j = t.zj % p.J;
  t.h0 = 2 * hp;
  t.two = (t.h0 + 1) < p.Hq;
  t.hk0 = t.h0 / p.G;
  t.hk1 = t.two ? (t.h0 + 1) / p.G : t.hk0;
  t.share = t.two && (t.hk1 == t.hk0);
  return t;
}
__device__ __forceinline__ unsigned q_slot_mask(const BwdQParams& p, int zj, int lane, int* my_idx) {
  int idx = -1;
  if (lane < p.K) idx = p.indices[(long long)zj * p.K + lane];
  *my_idx = idx;
  return __ballot_sync(0xffffffffu, idx >= 0 && idx < p.C);
}

__device__ void q_producer(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane) {
  using namespace qk;
  uint32_t ucnt = 0, kvcnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const QUnit t = decode_qunit(p, u);
    int my_idx;
    const unsigned mask = q_slot_mask(p, t.zj, lane, &my_idx);
    if (mask == 0) continue;
    const uint32_t qb = ucnt & 1;
    if (lane == 0) {
      ok = mbar_wait_bounded(&bars[QDO_EMPTY + qb], ((ucnt >> 1) & 1) ^ 1, abort_flag);
      if (ok) {
        uint8_t* base = smem + OFF_QDO + qb * 4 * TILE_BYTES;
        mbar_arrive_expect_tx(&bars[QDO_FULL + qb], (t.two ? 4 : 2) * TILE_BYTES);
        tma_load_5d(base, &p.tm_q, &bars[QDO_FULL + qb], 0, 0, t.h0, t.j, t.n);
        tma_load_5d(base + 2 * TILE_BYTES, &p.tm_do, &bars[QDO_FULL + qb], 0, 0, t.h0, t.j, t.n);
        if (t.two) {
          tma_load_5d(base + TILE_BYTES, &p.tm_q, &bars[QDO_FULL + qb], 0, 0, t.h0 + 1, t.j, t.n);
          tma_load_5d(base + 3 * TILE_BYTES, &p.tm_do, &bars[QDO_FULL + qb], 0, 0, t.h0 + 1, t.j, t.n);
        }
      }
    }
    ++ucnt;
    unsigned m = mask;
    while (m && ok) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      const int idx = __shfl_sync(0xffffffffu, my_idx, k);
      const uint32_t st = kvcnt % NSTAGE;
      if (lane == 0) {
        ok = mbar_wait_bounded(&bars[KV_EMPTY + st], ((kvcnt / NSTAGE) & 1) ^ 1, abort_flag);
        if (ok) {
          const bool both = t.two && !t.share;
          uint8_t* base = smem + OFF_KV + st * 4 * TILE_BYTES;
          mbar_arrive_expect_tx(&bars[KV_FULL + st], (both ? 4 : 2) * TILE_BYTES);
          tma_load_5d(base, &p.tm_k, &bars[KV_FULL + st], 0, 0, t.hk0, idx, t.n);
          tma_load_5d(base + 2 * TILE_BYTES, &p.tm_v, &bars[KV_FULL + st], 0, 0, t.hk0, idx, t.n);
          if (both) {
            tma_load_5d(base + TILE_BYTES, &p.tm_k, &bars[KV_FULL + st], 0, 0, t.hk1, idx, t.n);
            tma_load_5d(base + 3 * TILE_BYTES, &p.tm_v, &bars[KV_FULL + st], 0, 0, t.hk1, idx, t.n);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
      ++kvcnt;
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
  }
  if (lane == 0 && *abort_flag) {      // drain this lane's copies in flight (bounded)
    for (uint32_t back = 0; back < NSTAGE && back < kvcnt; ++back) {
      const uint32_t g = kvcnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[KV_FULL + g % NSTAGE], (g / NSTAGE) & 1)) break;
    }
    for (uint32_t back = 0; back < 2 && back < ucnt; ++back) {
      const uint32_t g = ucnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[QDO_FULL + (g & 1)], (g >> 1) & 1)) break;
    }
  }
}

__device__ void q_mma(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                      uint32_t tmem_base) {
  using namespace qk;
  uint32_t ucnt = 0, gcnt = 0;
  bool ok = true;
  const uint32_t sQDO = smem_u32(smem + OFF_QDO), sKV = smem_u32(smem + OFF_KV), sDS = smem_u32(smem + OFF_DS);
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const QUnit t = decode_qunit(p, u);
    int my_idx;
    const int nv = __popc(q_slot_mask(p, t.zj, lane, &my_idx));
    if (nv == 0) continue;
    if (lane == 0) {
      const uint32_t qb = ucnt & 1, ob = ucnt & 1;
      const int ntile = t.two ? 2 : 1;
      const uint32_t b_off = (t.two && !t.share) ? TILE_BYTES : 0;
      ok = mbar_wait_bounded(&bars[QDO_FULL + qb], (ucnt >> 1) & 1, abort_flag) &&
           mbar_wait_bounded(&bars[DQ_EMPTY + ob], ((ucnt >> 1) & 1) ^ 1, abort_flag);
      auto issue_sp = [&](uint32_t g) -> bool {
        const uint32_t st = g % NSTAGE, sb = g & 1;
        if (!mbar_wait_bounded(&bars[KV_FULL + st], (g / NSTAGE) & 1, abort_flag)) return false;
        if (!mbar_wait_bounded(&bars[SP_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        for (int tl = 0; tl < ntile; ++tl) {
          const uint32_t lane_off = tl ? LANE16 : 0u;
          const uint32_t qbase = sQDO + qb * 4 * TILE_BYTES + tl * TILE_BYTES;
          const uint32_t kbase = sKV + st * 4 * TILE_BYTES + (tl ? b_off : 0);
          mma_tile(tmem_base + COL_S + sb * 64 + lane_off, umma_desc_sw128(qbase), umma_desc_sw128(kbase), IDESC_KK,
                   STEP_K, STEP_K, false);
          mma_tile(tmem_base + COL_DP + sb * 64 + lane_off, umma_desc_sw128(qbase + 2 * TILE_BYTES),
                   umma_desc_sw128(kbase + 2 * TILE_BYTES), IDESC_KK, STEP_K, STEP_K, false);
        }
        umma_commit(&bars[SP_FULL + sb]);
        return true;
      };
      if (ok) ok = issue_sp(gcnt);
      for (int i = 0; i < nv && ok; ++i) {
        const uint32_t g = gcnt + i;
        if (i + 1 < nv) ok = issue_sp(g + 1);
        else umma_commit(&bars[QDO_EMPTY + qb]);
        if (!ok) break;
        const uint32_t st = g % NSTAGE, sb = g & 1;
        ok = mbar_wait_bounded(&bars[DS_FULL + sb], (g >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int tl = 0; tl < ntile; ++tl)     // dQ += dS K_k : A = dS (K-major), B = K_k (MN-major)
          mma_tile(tmem_base + COL_DQ + ob * 64 + (tl ? LANE16 : 0u),
                   umma_desc_sw128(sDS + sb * 2 * TILE_BYTES + tl * TILE_BYTES),
                   umma_desc_sw128(sKV + st * 4 * TILE_BYTES + (tl ? b_off : 0)), IDESC_KM, STEP_K, STEP_MN, i > 0);
        umma_commit(&bars[DS_EMPTY + sb]);
        umma_commit(&bars[KV_EMPTY + st]);
      }
      if (ok) umma_commit(&bars[DQ_FULL + ob]);
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    ++ucnt; gcnt += nv;
  }
}

__device__ void q_worker(const BwdQParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int warp,
                         int lane, uint32_t tmem_base) {
  using namespace qk;
  const int tile = lane >> 4;
  const int row = warp * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
  float* dws = reinterpret_cast<float*>(smem + OFF_DW);
  uint32_t ucnt = 0, gcnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const QUnit t = decode_qunit(p, u);
    const int h = t.h0 + tile;
    const bool live = h < p.Hq;
    int my_idx;
    const unsigned mask = q_slot_mask(p, t.zj, lane, &my_idx);
    const float my_w = lane < p.K ? p.weights[(long long)t.zj * p.K + lane] : 0.f;
    __nv_bfloat16* dq_row = p.dq + t.n * p.dqs[0] + t.j * p.dqs[1] + h * p.dqs[2] + row * p.dqs[3];
    float* dwp = p.dw_part + ((long long)t.zj * p.Hq + t.h0) * p.K;          // [tile][k] via + tile*K
    if (mask == 0) {
      if (live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(dq_row)[c] = z;
      }
      const int tid = warp * 32 + lane;
      if (tid < 2 * p.K && (t.h0 + tid / p.K) < p.Hq) dwp[tid] = 0.f;
      continue;
    }
    const uint32_t ob = ucnt & 1;
    float* dws_u = dws + (ucnt & 1) * (32 * 2 * 4);
    const float* lse_base = p.lse + ((long long)t.zj * p.Hq + (live ? h : t.h0)) * p.K * 64 + row;
    unsigned m = mask;
    while (m) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      const float w = __shfl_sync(0xffffffffu, my_w, k);
      const float lse = lse_base[k * 64];
      const uint32_t g = gcnt, sb = g & 1;
      ok = mbar_wait_bounded(&bars[SP_FULL + sb], (g >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[64], dp[64];
      tmem_ld_32x32b_x32(tlane + COL_S + sb * 64, s);
      tmem_ld_32x32b_x32(tlane + COL_S + sb * 64 + 32, s + 32);
      tmem_ld_32x32b_x32(tlane + COL_DP + sb * 64, dp);
      tmem_ld_32x32b_x32(tlane + COL_DP + sb * 64 + 32, dp + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars[SP_EMPTY + sb]);
      ok = mbar_wait_bounded(&bars[DS_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      uint8_t* ds_row = smem + OFF_DS + sb * 2 * TILE_BYTES + tile * TILE_BYTES + row * 128;
      float di = row_backward(s, dp, lse, p.c2, w, nullptr, ds_row, row);
      fence_proxy_async_smem();
      mbar_arrive(&bars[DS_FULL + sb]);
      // dw: sum of Di over the 16 rows this warp holds of each tile
#pragma unroll
      for (int of = 8; of > 0; of >>= 1) di += __shfl_xor_sync(0xffffffffu, di, of);
      if ((lane & 15) == 0) dws_u[(k * 2 + tile) * 4 + warp] = di;
      ++gcnt;
    }
    if (!ok) break;
    named_barrier_128();
    {
      const int tid = warp * 32 + lane;
      if (tid < 2 * p.K) {
        const int tl = tid / p.K, k = tid % p.K;
        if (t.h0 + tl < p.Hq) {
          float v = 0.f;
          if ((mask >> k) & 1) {
            const float* src = dws_u + (k * 2 + tl) * 4;
            v = ((src[0] + src[1]) + src[2]) + src[3];
          }
          dwp[tl * p.K + k] = v;
        }
      }
    }
    ok = mbar_wait_bounded(&bars[DQ_FULL + ob], (ucnt >> 1) & 1, abort_flag);
    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
    tc_fence_after();
    uint32_t acc[64];
    tmem_ld_32x32b_x32(tlane + COL_DQ + ob * 64, acc);
    tmem_ld_32x32b_x32(tlane + COL_DQ + ob * 64 + 32, acc + 32);
    tmem_ld_wait();
    tc_fence_before();
    mbar_arrive(&bars[DQ_EMPTY + ob]);
    if (live) store_row_bf16(dq_row, acc, p.sm_scale);
    ++ucnt;
  }
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
      mbar_init(&bars[SP_FULL + i], 1); mbar_init(&bars[SP_EMPTY + i], 128);
      mbar_init(&bars[DS_FULL + i], 128); mbar_init(&bars[DS_EMPTY + i], 1);
      mbar_init(&bars[DQ_FULL + i], 1); mbar_init(&bars[DQ_EMPTY + i], 128);
    }
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&bars[KV_FULL + i], 1); mbar_init(&bars[KV_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_do); tma_prefetch_desc(&p.tm_k); tma_prefetch_desc(&p.tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 4) q_worker(p, smem, bars, abort_flag, warp, lane, tmem_base);
  else if (warp == 4) q_producer(p, smem, bars, abort_flag, lane);
  else q_mma(p, smem, bars, abort_flag, lane, tmem_base);
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

// =============================================================================================
// kv-major kernel: dK, dV
// =============================================================================================
namespace kv {
constexpr int OFF_KV = 0;                                    // [2 bufs][Ka Kb Va Vb]
constexpr int OFF_QDO = OFF_KV + 2 * 4 * TILE_BYTES;         // [NSTAGE][Qa Qb dOa dOb]
constexpr int OFF_PDS = OFF_QDO + NSTAGE * 4 * TILE_BYTES;   // [2 bufs][Pwa Pwb dSa dSb]
constexpr int OFF_BAR = OFF_PDS + 2 * 4 * TILE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
enum Bar { KV_FULL = 0, KV_EMPTY = 2, QDO_FULL = 4, QDO_EMPTY = 4 + NSTAGE, SP_FULL = 4 + 2 * NSTAGE,
           SP_EMPTY = SP_FULL + 2, PDS_FULL = SP_EMPTY + 2, PDS_EMPTY = PDS_FULL + 2, ACC_FULL = PDS_EMPTY + 2,
           ACC_EMPTY = ACC_FULL + 2, NUM_BARS = ACC_EMPTY + 2 };
constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DK = 256, COL_DV = 384;   // each double-buffered, 64 columns
}  // namespace kv

struct BwdKvParams {
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  const float* weights;
  const float* lse;
  const int* offsets;
  const unsigned long long* sorted_keys;
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int32_t* status;
  long long dks[4], dvs[4];
  long long units;
  int N, J, Hq, Hkv, G, K, C, HP;
  float c2, sm_scale;
};

struct KvUnit { int nc, n, c, hk0, two, beg, end; };
__device__ __forceinline__ KvUnit decode_kvunit(const BwdKvParams& p, long long u) {
  KvUnit t;
  t.nc = (int)(u / p.HP);
  const int hp = (int)(u % p.HP);
  t.n = t.nc / p.C; t.c = t.nc % p.C;
  t.hk0 = 2 * hp;
  t.two = (t.hk0 + 1) < p.Hkv;
  t.beg = p.offsets[t.nc];
  t.end = p.offsets[t.nc + 1];
  return t;
}

__device__ void kv_producer(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag) {
  using namespace kv;
  uint32_t ucnt = 0, icnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const KvUnit t = decode_kvunit(p, u);
    if (t.end == t.beg) continue;
    const uint32_t kb = ucnt & 1;
    ok = mbar_wait_bounded(&bars[KV_EMPTY + kb], ((ucnt >> 1) & 1) ^ 1, abort_flag);
    if (!ok) break;
    {
      uint8_t* base = smem + OFF_KV + kb * 4 * TILE_BYTES;
      mbar_arrive_expect_tx(&bars[KV_FULL + kb], (t.two ? 4 : 2) * TILE_BYTES);
      tma_load_5d(base, &p.tm_k, &bars[KV_FULL + kb], 0, 0, t.hk0, t.c, t.n);
      tma_load_5d(base + 2 * TILE_BYTES, &p.tm_v, &bars[KV_FULL + kb], 0, 0, t.hk0, t.c, t.n);
      if (t.two) {
        tma_load_5d(base + TILE_BYTES, &p.tm_k, &bars[KV_FULL + kb], 0, 0, t.hk0 + 1, t.c, t.n);
        tma_load_5d(base + 3 * TILE_BYTES, &p.tm_v, &bars[KV_FULL + kb], 0, 0, t.hk0 + 1, t.c, t.n);
      }
    }
    ++ucnt;
    for (int e = t.beg; e < t.end && ok; ++e) {
      const int entry = (int)(p.sorted_keys[e] & 0xffffffffull);
      const int j = entry / p.K;
      for (int gi = 0; gi < p.G && ok; ++gi) {
        const uint32_t st = icnt % NSTAGE;
        ok = mbar_wait_bounded(&bars[QDO_EMPTY + st], ((icnt / NSTAGE) & 1) ^ 1, abort_flag);
        if (!ok) break;
        uint8_t* base = smem + OFF_QDO + st * 4 * TILE_BYTES;
        const int ha = t.hk0 * p.G + gi, hb = (t.hk0 + 1) * p.G + gi;
        mbar_arrive_expect_tx(&bars[QDO_FULL + st], (t.two ? 4 : 2) * TILE_BYTES);
        tma_load_5d(base, &p.tm_q, &bars[QDO_FULL + st], 0, 0, ha, j, t.n);
        tma_load_5d(base + 2 * TILE_BYTES, &p.tm_do, &bars[QDO_FULL + st], 0, 0, ha, j, t.n);
        if (t.two) {
          tma_load_5d(base + TILE_BYTES, &p.tm_q, &bars[QDO_FULL + st], 0, 0, hb, j, t.n);
          tma_load_5d(base + 3 * TILE_BYTES, &p.tm_do, &bars[QDO_FULL + st], 0, 0, hb, j, t.n);
        }
        ++icnt;
      }
    }
  }
  if (*abort_flag) {
    for (uint32_t back = 0; back < NSTAGE && back < icnt; ++back) {
      const uint32_t g = icnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[QDO_FULL + g % NSTAGE], (g / NSTAGE) & 1)) break;
    }
    for (uint32_t back = 0; back < 2 && back < ucnt; ++back) {
      const uint32_t g = ucnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[KV_FULL + (g & 1)], (g >> 1) & 1)) break;
    }
  }
}

__device__ void kv_mma(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag,
                       uint32_t tmem_base) {
  using namespace kv;
  uint32_t ucnt = 0, icnt = 0;
  bool ok = true;
  const uint32_t sKV = smem_u32(smem + OFF_KV), sQDO = smem_u32(smem + OFF_QDO), sPDS = smem_u32(smem + OFF_PDS);
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const KvUnit t = decode_kvunit(p, u);
    const int niter = (t.end - t.beg) * p.G;
    if (niter == 0) continue;
    const uint32_t kb = ucnt & 1, ob = ucnt & 1;
    const int ntile = t.two ? 2 : 1;
    ok = mbar_wait_bounded(&bars[KV_FULL + kb], (ucnt >> 1) & 1, abort_flag) &&
         mbar_wait_bounded(&bars[ACC_EMPTY + ob], ((ucnt >> 1) & 1) ^ 1, abort_flag);
    auto issue_sp = [&](uint32_t g) -> bool {
      const uint32_t st = g % NSTAGE, sb = g & 1;
      if (!mbar_wait_bounded(&bars[QDO_FULL + st], (g / NSTAGE) & 1, abort_flag)) return false;
      if (!mbar_wait_bounded(&bars[SP_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag)) return false;
      tc_fence_after();
      for (int tl = 0; tl < ntile; ++tl) {
        const uint32_t lane_off = tl ? LANE16 : 0u;
        const uint32_t qbase = sQDO + st * 4 * TILE_BYTES + tl * TILE_BYTES;
        const uint32_t kbase = sKV + kb * 4 * TILE_BYTES + tl * TILE_BYTES;
        mma_tile(tmem_base + COL_S + sb * 64 + lane_off, umma_desc_sw128(qbase), umma_desc_sw128(kbase), IDESC_KK,
                 STEP_K, STEP_K, false);
        mma_tile(tmem_base + COL_DP + sb * 64 + lane_off, umma_desc_sw128(qbase + 2 * TILE_BYTES),
                 umma_desc_sw128(kbase + 2 * TILE_BYTES), IDESC_KK, STEP_K, STEP_K, false);
      }
      umma_commit(&bars[SP_FULL + sb]);
      return true;
    };
    if (ok) ok = issue_sp(icnt);
    for (int i = 0; i < niter && ok; ++i) {
      const uint32_t g = icnt + i;
      if (i + 1 < niter) ok = issue_sp(g + 1);
      else umma_commit(&bars[KV_EMPTY + kb]);
      if (!ok) break;
      const uint32_t st = g % NSTAGE, sb = g & 1;
      ok = mbar_wait_bounded(&bars[PDS_FULL + sb], (g >> 1) & 1, abort_flag);
      if (!ok) break;
      tc_fence_after();
      for (int tl = 0; tl < ntile; ++tl) {
        const uint32_t lane_off = tl ? LANE16 : 0u;
        const uint32_t pbase = sPDS + sb * 4 * TILE_BYTES + tl * TILE_BYTES;
        const uint32_t qbase = sQDO + st * 4 * TILE_BYTES + tl * TILE_BYTES;
        // dV += (w P)^T dO : A = Pw read transposed (MN-major), B = dO (MN-major)
        mma_tile(tmem_base + COL_DV + ob * 64 + lane_off, umma_desc_sw128(pbase),
                 umma_desc_sw128(qbase + 2 * TILE_BYTES), IDESC_MM, STEP_MN, STEP_MN, i > 0);
        // dK += dS^T Q
        mma_tile(tmem_base + COL_DK + ob * 64 + lane_off, umma_desc_sw128(pbase + 2 * TILE_BYTES),
                 umma_desc_sw128(qbase), IDESC_MM, STEP_MN, STEP_MN, i > 0);
      }
      umma_commit(&bars[PDS_EMPTY + sb]);
      umma_commit(&bars[QDO_EMPTY + st]);
    }
    if (ok) umma_commit(&bars[ACC_FULL + ob]);
    ++ucnt; icnt += niter;
  }
}

__device__ void kv_worker(const BwdKvParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int warp,
                          int lane, uint32_t tmem_base) {
  using namespace kv;
  const int tile = lane >> 4;
  const int row = warp * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
  uint32_t ucnt = 0, icnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const KvUnit t = decode_kvunit(p, u);
    const int hk = t.hk0 + tile;
    const bool live = hk < p.Hkv;
    __nv_bfloat16* dk_row = p.dk + t.n * p.dks[0] + t.c * p.dks[1] + row * p.dks[2] + hk * p.dks[3];
    __nv_bfloat16* dv_row = p.dv + t.n * p.dvs[0] + t.c * p.dvs[1] + row * p.dvs[2] + hk * p.dvs[3];
    if (t.end == t.beg) {
      if (live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int c = 0; c < 8; ++c) { reinterpret_cast<uint4*>(dk_row)[c] = z; reinterpret_cast<uint4*>(dv_row)[c] = z; }
      }
      continue;
    }
    const uint32_t ob = ucnt & 1;
    for (int e = t.beg; e < t.end && ok; ++e) {
      const int entry = (int)(p.sorted_keys[e] & 0xffffffffull);
      const int j = entry / p.K, k = entry % p.K;
      const long long zj = (long long)t.n * p.J + j;
      const float w = p.weights[zj * p.K + k];
      for (int gi = 0; gi < p.G; ++gi) {
        const int h = (live ? hk : t.hk0) * p.G + gi;
        const float lse = p.lse[((zj * p.Hq + h) * p.K + k) * 64 + row];
        const uint32_t g = icnt, sb = g & 1;
        ok = mbar_wait_bounded(&bars[SP_FULL + sb], (g >> 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        tc_fence_after();
        uint32_t s[64], dp[64];
        tmem_ld_32x32b_x32(tlane + COL_S + sb * 64, s);
        tmem_ld_32x32b_x32(tlane + COL_S + sb * 64 + 32, s + 32);
        tmem_ld_32x32b_x32(tlane + COL_DP + sb * 64, dp);
        tmem_ld_32x32b_x32(tlane + COL_DP + sb * 64 + 32, dp + 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars[SP_EMPTY + sb]);
        ok = mbar_wait_bounded(&bars[PDS_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag);
        if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
        uint8_t* base = smem + OFF_PDS + sb * 4 * TILE_BYTES + tile * TILE_BYTES + row * 128;
        row_backward(s, dp, lse, p.c2, w, base, base + 2 * TILE_BYTES, row);
        fence_proxy_async_smem();
        mbar_arrive(&bars[PDS_FULL + sb]);
        ++icnt;
      }
    }
    if (!ok) break;
    ok = mbar_wait_bounded(&bars[ACC_FULL + ob], (ucnt >> 1) & 1, abort_flag);
    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
    tc_fence_after();
    uint32_t acc[64];
    tmem_ld_32x32b_x32(tlane + COL_DK + ob * 64, acc);
    tmem_ld_32x32b_x32(tlane + COL_DK + ob * 64 + 32, acc + 32);
    tmem_ld_wait();
    if (live) store_row_bf16(dk_row, acc, p.sm_scale);
    tmem_ld_32x32b_x32(tlane + COL_DV + ob * 64, acc);
    tmem_ld_32x32b_x32(tlane + COL_DV + ob * 64 + 32, acc + 32);
    tmem_ld_wait();
    tc_fence_before();
    mbar_arrive(&bars[ACC_EMPTY + ob]);
    if (live) store_row_bf16(dv_row, acc, 1.0f);
    ++ucnt;
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
bwd_kv_tc_kernel(const __grid_constant__ BwdKvParams p) {
  using namespace kv;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[KV_FULL + i], 1); mbar_init(&bars[KV_EMPTY + i], 1);
      mbar_init(&bars[SP_FULL + i], 1); mbar_init(&bars[SP_EMPTY + i], 128);
      mbar_init(&bars[PDS_FULL + i], 128); mbar_init(&bars[PDS_EMPTY + i], 1);
      mbar_init(&bars[ACC_FULL + i], 1); mbar_init(&bars[ACC_EMPTY + i], 128);
    }
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&bars[QDO_FULL + i], 1); mbar_init(&bars[QDO_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_do); tma_prefetch_desc(&p.tm_k); tma_prefetch_desc(&p.tm_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (warp < 4) kv_worker(p, smem, bars, abort_flag, warp, lane, tmem_base);
  else if (warp == 4) { if (lane == 0) kv_producer(p, smem, bars, abort_flag); }
  else { if (lane == 0) kv_mma(p, smem, bars, abort_flag, tmem_base); }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

}  // namespace

bool bwd_tc_available() { return true; }

int launch_bwd_tc(const GcaBwdArgs& a, const Csr& csr, float* dw_part, cudaStream_t stream) {
  if (a.dtype != GCA_BF16 || a.S != 64 || a.L != 64 || a.D != 64 || a.K > 32) return GCA_ERR_ALGO;
  int dev = 0, sms = 0;
  GCA_CUDA_CHECK(cudaGetDevice(&dev));
  GCA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  CUtensorMap tm_q, tm_do, tm_k, tm_v;
  int rc;
  if ((rc = make_tile_map_5d(&tm_q, a.q, 64, 64, a.Hq, a.J, a.N, a.q_stride[3], a.q_stride[2], a.q_stride[1], a.q_stride[0]))) return rc;
  if ((rc = make_tile_map_5d(&tm_do, a.dout, 64, 64, a.Hq, a.J, a.N, a.do_stride[3], a.do_stride[2], a.do_stride[1], a.do_stride[0]))) return rc;
  if ((rc = make_tile_map_5d(&tm_k, a.k_cache, 64, 64, a.Hkv, a.C, a.N, a.k_stride[2], a.k_stride[3], a.k_stride[1], a.k_stride[0]))) return rc;
  if ((rc = make_tile_map_5d(&tm_v, a.v_cache, 64, 64, a.Hkv, a.C, a.N, a.v_stride[2], a.v_stride[3], a.v_stride[1], a.v_stride[0]))) return rc;
  const float c2 = a.sm_scale * GCA_LOG2E;
  {
    BwdKvParams p;
    p.tm_q = tm_q; p.tm_do = tm_do; p.tm_k = tm_k; p.tm_v = tm_v;
    p.weights = a.weights; p.lse = a.lse; p.offsets = csr.offsets; p.sorted_keys = csr.sorted_keys;
    p.dk = (__nv_bfloat16*)a.dk_cache; p.dv = (__nv_bfloat16*)a.dv_cache; p.status = a.status;
    for (int i = 0; i < 4; ++i) { p.dks[i] = a.dk_stride[i]; p.dvs[i] = a.dv_stride[i]; }
    p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
    p.HP = (a.Hkv + 1) / 2;
    p.units = (long long)a.N * a.C * p.HP;
    p.c2 = c2; p.sm_scale = a.sm_scale;
    if (p.units > 0) {
      GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_kv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kv::SMEM_BYTES));
      const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
      bwd_kv_tc_kernel<<<grid, NTHREADS, kv::SMEM_BYTES, stream>>>(p);
      GCA_CUDA_CHECK(cudaGetLastError());
    }
  }
  {
    BwdQParams p;
    p.tm_q = tm_q; p.tm_do = tm_do; p.tm_k = tm_k; p.tm_v = tm_v;
    p.indices = a.indices; p.weights = a.weights; p.lse = a.lse;
    p.dq = (__nv_bfloat16*)a.dq; p.dw_part = dw_part; p.status = a.status;
    for (int i = 0; i < 4; ++i) p.dqs[i] = a.dq_stride[i];
    p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
    p.HP = (a.Hq + 1) / 2;
    p.units = (long long)a.N * a.J * p.HP;
    p.c2 = c2; p.sm_scale = a.sm_scale;
    if (p.units > 0) {
      GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, qk::SMEM_BYTES));
      const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
      bwd_q_tc_kernel<<<grid, NTHREADS, qk::SMEM_BYTES, stream>>>(p);
      GCA_CUDA_CHECK(cudaGetLastError());
    }
  }
  return 0;
}

}  // namespace gca
