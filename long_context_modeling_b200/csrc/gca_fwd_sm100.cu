// GCA forward on the 5th-generation tensor cores (tcgen05 + TMEM), bf16, S = L = D = 64.
//
// Work unit: one (sequence n, query chunk j, PAIR of q heads).  A 64-row MMA writes only
// 16 of the 32 TMEM lanes of each lane quarter, so two 64-row tiles are interleaved
// (head A in lanes 0-15, head B in lanes 16-31 of every quarter): each of the 128 softmax
// threads then owns one complete row of one head, and row max / row sum need no shuffles.
//
// Per retrieved slot k (padding slots are skipped):
//   S   = Q K_k^T             tcgen05.mma  M=64 N=64 K=64, Q and K_k K-major in smem
//   P   = w_k * softmax(S)    one thread per row: tcgen05.ld, exp2, scale by w_k / l, bf16
//   O  += P V_k               tcgen05.mma  with V_k as MN-major B operand; the K slots
//                             accumulate in ONE TMEM tile, which fuses the weighted merge
// K_k / V_k tiles are fetched straight from the chunk cache by TMA with the retrieved chunk
// index as a tensor coordinate (no gathered copy exists).  Softmax of a slot needs only
// that slot's 64 keys, so there is no running rescale.
//
// CTA = 6 warps: warps 0-3 softmax + epilogue, warp 4 TMA producer, warp 5 MMA issuer.
// CTAs are persistent and walk the units in (n, j, head pair) order so that concurrently
// running CTAs touch the cache of few sequences (L2 reuse of chunks retrieved many times).
// Every mbarrier wait is bounded; on expiry the CTA flags GCA_STATUS_TIMEOUT and unwinds.
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
constexpr int TMEM_COLS = 256;          // S0 | S1 | O0 | O1, 64 columns each

constexpr int OFF_Q = 0;                              // [2 bufs][2 tiles]
constexpr int OFF_KV = OFF_Q + 4 * TILE_BYTES;        // [NSTAGE][Ka Kb Va Vb]
constexpr int OFF_P = OFF_KV + NSTAGE * 4 * TILE_BYTES;   // [2 bufs][2 tiles]
constexpr int OFF_BAR = OFF_P + 4 * TILE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;      // + alignment slack

enum Bar { Q_FULL = 0, Q_EMPTY = 2, KV_FULL = 4, KV_EMPTY = 4 + NSTAGE, S_FULL = 4 + 2 * NSTAGE,
           S_EMPTY = S_FULL + 2, P_FULL = S_EMPTY + 2, P_EMPTY = P_FULL + 2, O_FULL = P_EMPTY + 2,
           O_EMPTY = O_FULL + 2, NUM_BARS = O_EMPTY + 2 };

constexpr uint32_t IDESC_S = umma_idesc_bf16(64, 64, 0, 0);
constexpr uint32_t IDESC_PV = umma_idesc_bf16(64, 64, 0, 1);

struct FwdTcParams {
  CUtensorMap tm_q, tm_k, tm_v;
  const int32_t* indices;
  const float* weights;
  __nv_bfloat16* out;
  float* lse;
  int32_t* status;
  long long os[4];
  long long units;
  int N, J, Hq, Hkv, G, K, C, HP;
  int pair;                 // 1: a unit is a pair of q heads; 0: a single head (debug knob)
  float c2;
  float off_by_one;
};

struct Unit {
  int zj, n, j, h0, two, hk0, hk1, share;
};
__device__ __forceinline__ Unit decode_unit(const FwdTcParams& p, long long u) {
  Unit t;
  t.zj = (int)(u / p.HP);
  const int hp = (int)(u % p.HP);
  t.n = t.zj / p.J; t.j = t.zj % p.J;
  t.h0 = p.pair ? 2 * hp : hp;
  t.two = p.pair && (t.h0 + 1) < p.Hq;
  t.hk0 = t.h0 / p.G;
  t.hk1 = t.two ? (t.h0 + 1) / p.G : t.hk0;
  t.share = t.two && (t.hk1 == t.hk0);
  return t;
}
// bit k set when slot k of (zj) holds a usable chunk index; also returns this lane's index
__device__ __forceinline__ unsigned slot_mask(const FwdTcParams& p, int zj, int lane, int* my_idx, bool* bad) {
  int idx = -1;
  if (lane < p.K) idx = p.indices[(long long)zj * p.K + lane];
  *my_idx = idx;
  *bad = __any_sync(0xffffffffu, idx >= p.C);
  return __ballot_sync(0xffffffffu, idx >= 0 && idx < p.C);
}

// ----------------------------------------------------------------------------- producer
__device__ void producer_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane) {
  uint32_t qcnt = 0, kvcnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const Unit t = decode_unit(p, u);
    int my_idx; bool bad;
    const unsigned mask = slot_mask(p, t.zj, lane, &my_idx, &bad);
    if (mask == 0) continue;
    const uint32_t qb = qcnt & 1;
    if (lane == 0) {
      ok = mbar_wait_bounded(&bars[Q_EMPTY + qb], ((qcnt >> 1) & 1) ^ 1, abort_flag);
      if (ok) {
        mbar_arrive_expect_tx(&bars[Q_FULL + qb], t.two ? 2 * TILE_BYTES : TILE_BYTES);
        tma_load_5d(smem + OFF_Q + qb * 2 * TILE_BYTES, &p.tm_q, &bars[Q_FULL + qb], 0, 0, t.h0, t.j, t.n);
        if (t.two)
          tma_load_5d(smem + OFF_Q + qb * 2 * TILE_BYTES + TILE_BYTES, &p.tm_q, &bars[Q_FULL + qb], 0, 0, t.h0 + 1, t.j, t.n);
      }
    }
    ++qcnt;
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
          mbar_arrive_expect_tx(&bars[KV_FULL + st], both ? 4 * TILE_BYTES : 2 * TILE_BYTES);
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
  // If anybody gave up, wait (bounded) for the copies this lane still has in flight so no
  // bulk copy can land in shared memory after the CTA has exited.
  if (lane == 0 && *abort_flag) {
    for (uint32_t back = 0; back < NSTAGE && back < kvcnt; ++back) {
      const uint32_t g = kvcnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[KV_FULL + g % NSTAGE], (g / NSTAGE) & 1)) break;
    }
    for (uint32_t back = 0; back < 2 && back < qcnt; ++back) {
      const uint32_t g = qcnt - 1 - back;
      for (int i = 0; i < (1 << 20); ++i)
        if (mbar_try_wait(&bars[Q_FULL + (g & 1)], (g >> 1) & 1)) break;
    }
  }
}

// ----------------------------------------------------------------------------- MMA issuer
__device__ void mma_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                         uint32_t tmem_base) {
  uint32_t qcnt = 0, gcnt = 0, ocnt = 0;
  bool ok = true;
  const uint32_t sQ = smem_u32(smem + OFF_Q), sKV = smem_u32(smem + OFF_KV), sP = smem_u32(smem + OFF_P);
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const Unit t = decode_unit(p, u);
    int my_idx; bool bad;
    const unsigned mask = slot_mask(p, t.zj, lane, &my_idx, &bad);
    const int nv = __popc(mask);
    if (nv == 0) continue;
    if (lane == 0) {
      const uint32_t qb = qcnt & 1, ob = ocnt & 1;
      const int ntile = t.two ? 2 : 1;
      const uint32_t b_off = (t.two && !t.share) ? TILE_BYTES : 0;   // where tile B's K/V sit
      ok = mbar_wait_bounded(&bars[Q_FULL + qb], (qcnt >> 1) & 1, abort_flag) &&
           mbar_wait_bounded(&bars[O_EMPTY + ob], ((ocnt >> 1) & 1) ^ 1, abort_flag);

      auto issue_s = [&](uint32_t g) -> bool {
        const uint32_t st = g % NSTAGE, sb = g & 1;
        if (!mbar_wait_bounded(&bars[KV_FULL + st], (g / NSTAGE) & 1, abort_flag)) return false;
        if (!mbar_wait_bounded(&bars[S_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag)) return false;
        tc_fence_after();
        for (int tl = 0; tl < ntile; ++tl) {
          const uint64_t a = umma_desc_sw128(sQ + qb * 2 * TILE_BYTES + tl * TILE_BYTES);
          const uint64_t b = umma_desc_sw128(sKV + st * 4 * TILE_BYTES + (tl ? b_off : 0));
          const uint32_t d = tmem_base + sb * 64 + (tl ? (16u << 16) : 0u);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(d, a + kk * 2, b + kk * 2, IDESC_S, kk > 0);
        }
        umma_commit(&bars[S_FULL + sb]);
        return true;
      };

      if (ok) ok = issue_s(gcnt);
      for (int i = 0; i < nv && ok; ++i) {
        const uint32_t g = gcnt + i;
        if (i + 1 < nv) ok = issue_s(g + 1);
        else umma_commit(&bars[Q_EMPTY + qb]);      // every S MMA of the unit has been issued
        if (!ok) break;
        const uint32_t st = g % NSTAGE, sb = g & 1;
        ok = mbar_wait_bounded(&bars[P_FULL + sb], (g >> 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        for (int tl = 0; tl < ntile; ++tl) {
          const uint64_t a = umma_desc_sw128(sP + sb * 2 * TILE_BYTES + tl * TILE_BYTES);
          const uint64_t b = umma_desc_sw128(sKV + st * 4 * TILE_BYTES + 2 * TILE_BYTES + (tl ? b_off : 0));
          const uint32_t d = tmem_base + 128 + ob * 64 + (tl ? (16u << 16) : 0u);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) umma_bf16_ss(d, a + kk * 2, b + kk * 128, IDESC_PV, (i > 0 || kk > 0));
        }
        umma_commit(&bars[P_EMPTY + sb]);
        umma_commit(&bars[KV_EMPTY + st]);
      }
      if (ok) umma_commit(&bars[O_FULL + ob]);
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    ++qcnt; ++ocnt; gcnt += nv;
  }
}

// ----------------------------------------------------------------------------- softmax + epilogue
__device__ void softmax_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int warp,
                             int lane, uint32_t tmem_base) {
  const int tile = lane >> 4;
  const int row = warp * 16 + (lane & 15);
  const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);
  uint8_t* sP = smem + OFF_P;
  uint32_t gcnt = 0, ocnt = 0;
  bool ok = true;
  for (long long u = blockIdx.x; u < p.units && ok; u += gridDim.x) {
    const Unit t = decode_unit(p, u);
    const int h = t.h0 + tile;
    const bool live = (tile == 0 || t.two) && h < p.Hq;
    int my_idx; bool bad;
    const unsigned mask = slot_mask(p, t.zj, lane, &my_idx, &bad);
    if (bad && p.status && warp == 0 && lane == 0) atomicOr(p.status, GCA_STATUS_BAD_INDEX);
    const float my_w = lane < p.K ? p.weights[(long long)t.zj * p.K + lane] : 0.f;
    float* lse_base = p.lse ? p.lse + ((long long)t.zj * p.Hq + h) * p.K * 64 + row : nullptr;
    if (lse_base && live)
      for (int k = 0; k < p.K; ++k)
        if (!((mask >> k) & 1)) lse_base[k * 64] = 0.f;
    __nv_bfloat16* orow = p.out + t.n * p.os[0] + t.j * p.os[1] + h * p.os[2] + row * p.os[3];
    if (mask == 0) {
      if (live) {
        const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(orow)[c] = z;
      }
      continue;
    }
    const uint32_t ob = ocnt & 1;
    unsigned m = mask;
    while (m) {
      const int k = __ffs(m) - 1;
      m &= m - 1;
      const float w = __shfl_sync(0xffffffffu, my_w, k);
      const uint32_t g = gcnt, sb = g & 1;
      ok = mbar_wait_bounded(&bars[S_FULL + sb], (g >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      uint32_t x[64];
      tmem_ld_32x32b_x32(tlane + sb * 64, x);
      tmem_ld_32x32b_x32(tlane + sb * 64 + 32, x + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars[S_EMPTY + sb]);

      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; ++c) mx = fmaxf(mx, __uint_as_float(x[c]));
      float mm = mx * p.c2;
      if (p.off_by_one > 0.f) mm = fmaxf(mm, 0.f);
      float l = 0.f;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float e = ex2_approx(fmaf(__uint_as_float(x[c]), p.c2, -mm));
        x[c] = __float_as_uint(e);
        l += e;
      }
      if (p.off_by_one > 0.f) l += p.off_by_one * ex2_approx(-mm);
      if (lse_base && live) lse_base[k * 64] = mm + __log2f(l);
      const float f = w / l;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c)
        pk[c] = pack_bf16x2(__uint_as_float(x[2 * c]) * f, __uint_as_float(x[2 * c + 1]) * f);

      ok = mbar_wait_bounded(&bars[P_EMPTY + sb], ((g >> 1) & 1) ^ 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      uint8_t* prow = sP + sb * 2 * TILE_BYTES + tile * TILE_BYTES + row * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(prow + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_proxy_async_smem();
      mbar_arrive(&bars[P_FULL + sb]);
      ++gcnt;
    }
    if (!ok) break;
    // epilogue: O tile -> bf16 -> global, one 128-byte row per thread
    ok = mbar_wait_bounded(&bars[O_FULL + ob], (ocnt >> 1) & 1, abort_flag);
    if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
    tc_fence_after();
    uint32_t o[64];
    tmem_ld_32x32b_x32(tlane + 128 + ob * 64, o);
    tmem_ld_32x32b_x32(tlane + 128 + ob * 64 + 32, o + 32);
    tmem_ld_wait();
    tc_fence_before();
    mbar_arrive(&bars[O_EMPTY + ob]);
    if (live) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 v;
        v.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]), __uint_as_float(o[8 * c + 1]));
        v.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]), __uint_as_float(o[8 * c + 3]));
        v.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]), __uint_as_float(o[8 * c + 5]));
        v.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]), __uint_as_float(o[8 * c + 7]));
        reinterpret_cast<uint4*>(orow)[c] = v;
      }
    }
    ++ocnt;
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
fwd_tc_kernel(const __grid_constant__ FwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[Q_FULL + i], 1); mbar_init(&bars[Q_EMPTY + i], 1);
      mbar_init(&bars[S_FULL + i], 1); mbar_init(&bars[S_EMPTY + i], 128);
      mbar_init(&bars[P_FULL + i], 128); mbar_init(&bars[P_EMPTY + i], 1);
      mbar_init(&bars[O_FULL + i], 1); mbar_init(&bars[O_EMPTY + i], 128);
    }
    for (int i = 0; i < NSTAGE; ++i) { mbar_init(&bars[KV_FULL + i], 1); mbar_init(&bars[KV_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == 4 && lane == 0) { tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_k); tma_prefetch_desc(&p.tm_v); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4) softmax_role(p, smem, bars, abort_flag, warp, lane, tmem_base);
  else if (warp == 4) producer_role(p, smem, bars, abort_flag, lane);
  else mma_role(p, smem, bars, abort_flag, lane, tmem_base);

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

}  // namespace

int launch_fwd_tc(const GcaFwdArgs& a, cudaStream_t stream) {
  if (a.dtype != GCA_BF16 || a.S != 64 || a.L != 64 || a.D != 64 || a.K > 32) return GCA_ERR_ALGO;
  FwdTcParams p;
  // q viewed as (d, s, h, j, n); caches as (d, l, h, c, n): box = one 64 x 64 tile
  int rc = make_tile_map_5d(&p.tm_q, a.q, 64, 64, a.Hq, a.J, a.N, a.q_stride[3], a.q_stride[2], a.q_stride[1], a.q_stride[0]);
  if (rc) return rc;
  rc = make_tile_map_5d(&p.tm_k, a.k_cache, 64, 64, a.Hkv, a.C, a.N, a.k_stride[2], a.k_stride[3], a.k_stride[1], a.k_stride[0]);
  if (rc) return rc;
  rc = make_tile_map_5d(&p.tm_v, a.v_cache, 64, 64, a.Hkv, a.C, a.N, a.v_stride[2], a.v_stride[3], a.v_stride[1], a.v_stride[0]);
  if (rc) return rc;
  p.indices = a.indices; p.weights = a.weights; p.out = (__nv_bfloat16*)a.out; p.lse = a.lse; p.status = a.status;
  for (int i = 0; i < 4; ++i) p.os[i] = a.o_stride[i];
  p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
  const char* pair_env = getenv("GCA_TC_PAIR");
  p.pair = (pair_env && pair_env[0] == '0') ? 0 : 1;
  p.HP = p.pair ? (a.Hq + 1) / 2 : a.Hq;
  p.units = (long long)a.N * a.J * p.HP;
  p.c2 = a.sm_scale * GCA_LOG2E;
  p.off_by_one = a.off_by_one;
  if (p.units == 0) return 0;
  int dev = 0, sms = 0;
  GCA_CUDA_CHECK(cudaGetDevice(&dev));
  GCA_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  GCA_CUDA_CHECK(cudaFuncSetAttribute(fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
  fwd_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace gca
