// GCA forward for a handful of query rows (autoregressive decode: 1 or 2 rows per
// sequence).  The work is a stream over K retrieved chunks x (K tile + V tile) per
// (sequence, kv head): HBM-bound, no tensor cores.  Two kernels: up to four rows per kv head (the
// model's decode step) take `decode_rows_kernel`, which streams the tiles through registers (see
// its comment); 5-16 rows take `decode_kernel`, described here.  Blocks are persistent (one per SM: each
// warp keeps a K and a V tile, 128 KB per block) and walk the (n, j, kv head) items; each warp
// owns whole slots and fetches its slot's two 8 KB tiles with two TMA copies (retrieved chunk
// index = tensor coordinate) onto two mbarriers of its own, so nothing is staged through
// registers.  As soon as a warp has scored its queries against the K tile it puts the K tile
// of its NEXT slot in flight -- of the next item when this one has no more slots for it -- and
// likewise the V tile after P.V: the loads of an item run under the arithmetic, the block-wide
// merge and the output store of the one before.  The K tile lands 128-byte-swizzled
// (conflict-free row reads), the V tile plain.  A warp scores the R = G*S query rows against
// the 64 keys (two keys per lane), normalises inside the warp and accumulates its weighted
// P.V in registers; the per-warp partial outputs are summed in warp order, so the result does
// not depend on scheduling.
#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace gca {

namespace {

using namespace sm100;

constexpr int T = 64;
constexpr int NWARPS = 8;
constexpr int TILE_BYTES = T * T * 2;      // one bf16 tile

__device__ __forceinline__ float bf_lo(unsigned v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(unsigned v) { return __uint_as_float(v & 0xffff0000u); }

struct DecParams {
  CUtensorMap tm_k, tm_v;
  const __nv_bfloat16* q;
  const int32_t* indices;
  const float* weights;
  __nv_bfloat16* out;
  int32_t* status;
  Geom g;
};

template <int R>
__global__ void __launch_bounds__(NWARPS * 32)
decode_kernel(const __grid_constant__ DecParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t* tile_k = smem + warp * 2 * TILE_BYTES;                                       // swizzled
  uint8_t* tile_v = tile_k + TILE_BYTES;                                                // plain
  float* sQ_all = reinterpret_cast<float*>(smem + NWARPS * 2 * TILE_BYTES);             // [2][R x 64] scaled queries
  float* part_all = sQ_all + 2 * R * T;                                                 // [2][NWARPS][R x 64] partial outputs
  uint64_t* bars = reinterpret_cast<uint64_t*>(part_all + 2 * NWARPS * R * T);          // [NWARPS][K, V]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 2 * NWARPS);
  const Geom& g = p.g;
  const int items = g.N * g.J * g.Hkv;
  const int rows = g.G * g.S;                                    // <= R
  const float c2 = g.sm_scale * GCA_LOG2E;
  uint64_t* bar_k = &bars[2 * warp];
  uint64_t* bar_v = &bars[2 * warp + 1];

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2 * NWARPS; ++i) mbar_init(&bars[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();

  // This warp's slots, in order: (item, k) with k = warp, warp + 8, ... < K, then the next item.
  // `cur` is the slot whose tiles are (or are about to be) in the buffers; idx < 0: no copy.
  struct Slot { int item, k, idx; };
  auto load_idx = [&](int item, int k) -> int {
    const int zj = item / g.Hkv;
    const int v = p.indices[(long long)zj * g.K + k];
    if (v >= g.C) { if (p.status && lane == 0) atomicOr(p.status, GCA_STATUS_BAD_INDEX); return -1; }
    return v;
  };
  auto next_slot = [&](const Slot& s) -> Slot {
    Slot t;
    t.item = s.item; t.k = s.k + NWARPS;
    if (t.k >= g.K) { t.item = s.item + (int)gridDim.x; t.k = warp; }
    t.idx = (t.item < items && t.k < g.K) ? load_idx(t.item, t.k) : -1;
    return t;
  };
  auto issue = [&](const Slot& s, bool is_v) {
    if (lane == 0) {
      const int zj = s.item / g.Hkv, hk = s.item - zj * g.Hkv;
      uint64_t* bar = is_v ? bar_v : bar_k;
      mbar_arrive_expect_tx(bar, TILE_BYTES);
      tma_load_5d(is_v ? tile_v : tile_k, is_v ? &p.tm_v : &p.tm_k, bar, 0, 0, hk, s.idx, zj / g.J);
    }
  };

  Slot cur;
  cur.item = blockIdx.x; cur.k = warp;
  cur.idx = (cur.item < items && cur.k < g.K) ? load_idx(cur.item, cur.k) : -1;
  bool in_k = false, in_v = false;               // a copy is in flight (or landed, unread) in the K / V buffer
  if (cur.idx >= 0) { issue(cur, false); issue(cur, true); in_k = in_v = true; }
  uint32_t ph_k = 0, ph_v = 0;
  bool ok = true;

  int par = 0;
  for (int item = blockIdx.x; item < items; item += gridDim.x, par ^= 1) {
    const int zj = item / g.Hkv, hk = item - zj * g.Hkv;
    const int n = zj / g.J, j = zj - n * g.J;
    float* sQ = sQ_all + par * R * T;
    float* part = part_all + par * NWARPS * R * T;
    for (int i = threadIdx.x; i < R * T; i += NWARPS * 32) {
      const int r = i >> 6, d = i & 63;
      float v = 0.f;
      if (r < rows) {
        const int gi = r / g.S, s = r % g.S;
        v = __bfloat162float(p.q[n * g.qs[0] + j * g.qs[1] + (hk * g.G + gi) * g.qs[2] + s * g.qs[3] + d]);
      }
      sQ[i] = v * c2;
    }
    __syncthreads();

    float o[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r) { o[r][0] = 0.f; o[r][1] = 0.f; }

    while (cur.item == item && cur.k < g.K) {
      const Slot nxt = next_slot(cur);           // its index load overlaps the waits below
      float pr[R][2];
      if (cur.idx >= 0 && ok) {
        const float w = p.weights[(long long)zj * g.K + cur.k];
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_k, ph_k, abort_flag));
        ph_k ^= 1;
        in_k = false;
        if (ok) {
#pragma unroll
          for (int r = 0; r < R; ++r) {
            pr[r][0] = pr[r][1] = 0.f;
            if (r >= rows) continue;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int pc = 0; pc < 8; ++pc) {
              const uint4 a = *reinterpret_cast<const uint4*>(tile_k + lane * 128 + ((pc ^ (lane & 7)) << 4));
              const uint4 b = *reinterpret_cast<const uint4*>(tile_k + (lane + 32) * 128 + ((pc ^ (lane & 7)) << 4));
              const float* qr = sQ + r * T + pc * 8;
              s0 = fmaf(qr[0], bf_lo(a.x), s0); s0 = fmaf(qr[1], bf_hi(a.x), s0);
              s0 = fmaf(qr[2], bf_lo(a.y), s0); s0 = fmaf(qr[3], bf_hi(a.y), s0);
              s0 = fmaf(qr[4], bf_lo(a.z), s0); s0 = fmaf(qr[5], bf_hi(a.z), s0);
              s0 = fmaf(qr[6], bf_lo(a.w), s0); s0 = fmaf(qr[7], bf_hi(a.w), s0);
              s1 = fmaf(qr[0], bf_lo(b.x), s1); s1 = fmaf(qr[1], bf_hi(b.x), s1);
              s1 = fmaf(qr[2], bf_lo(b.y), s1); s1 = fmaf(qr[3], bf_hi(b.y), s1);
              s1 = fmaf(qr[4], bf_lo(b.z), s1); s1 = fmaf(qr[5], bf_hi(b.z), s1);
              s1 = fmaf(qr[6], bf_lo(b.w), s1); s1 = fmaf(qr[7], bf_hi(b.w), s1);
            }
            float m = fmaxf(s0, s1);
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, of));
            if (g.off_by_one > 0.f) m = fmaxf(m, 0.f);
            float p0 = exp2f(s0 - m), p1 = exp2f(s1 - m);
            float l = p0 + p1;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) l += __shfl_xor_sync(0xffffffffu, l, of);
            if (g.off_by_one > 0.f) l += g.off_by_one * exp2f(-m);
            const float f = w / l;
            pr[r][0] = p0 * f; pr[r][1] = p1 * f;
          }
        }
      }
      // the K buffer has been read: the next slot's K tile goes in flight under the P.V below
      __syncwarp();
      if (nxt.idx >= 0 && ok) { issue(nxt, false); in_k = true; }
      if (cur.idx >= 0 && ok) {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded(bar_v, ph_v, abort_flag));
        ph_v ^= 1;
        in_v = false;
        if (ok) {
#pragma unroll
          for (int r = 0; r < R; ++r) {
            if (r >= rows) break;
            float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
            for (int key = 0; key < 32; ++key) {
              const float pa = __shfl_sync(0xffffffffu, pr[r][0], key);
              const float pb = __shfl_sync(0xffffffffu, pr[r][1], key);
              const unsigned va = *reinterpret_cast<const unsigned*>(tile_v + key * 128 + lane * 4);
              const unsigned vb = *reinterpret_cast<const unsigned*>(tile_v + (key + 32) * 128 + lane * 4);
              a0 = fmaf(pa, bf_lo(va), a0); a1 = fmaf(pa, bf_hi(va), a1);
              a0 = fmaf(pb, bf_lo(vb), a0); a1 = fmaf(pb, bf_hi(vb), a1);
            }
            o[r][0] += a0; o[r][1] += a1;
          }
        }
      }
      __syncwarp();
      if (nxt.idx >= 0 && ok) { issue(nxt, true); in_v = true; }
      cur = nxt;
    }
    // cross-warp sum in warp order
#pragma unroll
    for (int r = 0; r < R; ++r) {
      part[(warp * R + r) * T + 2 * lane] = o[r][0];
      part[(warp * R + r) * T + 2 * lane + 1] = o[r][1];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * T; i += NWARPS * 32) {
      const int r = i >> 6, d = i & 63;
      float t = 0.f;
#pragma unroll
      for (int wv = 0; wv < NWARPS; ++wv) t += part[(wv * R + r) * T + d];
      const int gi = r / g.S, s = r % g.S;
      p.out[n * g.os[0] + j * g.os[1] + (hk * g.G + gi) * g.os[2] + s * g.os[3] + d] = __float2bfloat16_rn(t);
    }
  }
  // a warp that gave up may still have copies in flight: wait for them (bounded) so nothing
  // lands in shared memory after the block has exited
  if (lane == 0) {
    if (in_k) for (int i = 0; i < (1 << 20); ++i) if (mbar_try_wait(bar_k, ph_k)) break;
    if (in_v) for (int i = 0; i < (1 << 20); ++i) if (mbar_try_wait(bar_v, ph_v)) break;
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

// ---------------------------------------------------------------------------------------------
// Up to four query rows per kv head (the model's decode step: one row): no shared-memory staging at
// all.  One CTA per (sequence, query chunk, kv head), one warp per retrieved slot (slots k = warp,
// warp + 8, ...).  A warp load covers FOUR key rows of the slot's tile (8 lanes x 16 bytes per
// 128-byte row); every 8-lane group owns a stream of 16 keys with its own online-softmax state, the
// loads run four steps ahead of the arithmetic in registers, and nothing is waited for except the
// data itself.  Registers are capped so that three CTAs share an SM: 32 sequences x
// 12 heads = 384 CTAs run as one wave, where the persistent TMA kernel below needs a ragged third
// round of its 148 CTAs.  The four streams of a warp, then the slots in slot order, are merged in a
// fixed order: the result does not depend on scheduling.
struct RowState { float m, l, acc[8]; };
__device__ __forceinline__ float ex2f(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void merge_state(RowState& a, float m2, float l2, const float* acc2) {
  const float m = fmaxf(a.m, m2);
  const float ca = (a.m == -INFINITY) ? 0.f : ex2f(a.m - m), cb = (m2 == -INFINITY) ? 0.f : ex2f(m2 - m);
  a.l = a.l * ca + l2 * cb;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.acc[i] = a.acc[i] * ca + acc2[i] * cb;
  a.m = m;
}

template <int R>
__global__ void __launch_bounds__(NWARPS * 32, R == 1 ? 3 : (R == 2 ? 2 : 1))
decode_rows_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc, const __nv_bfloat16* __restrict__ vc,
                   const int32_t* __restrict__ indices, const float* __restrict__ weights, __nv_bfloat16* __restrict__ out,
                   int32_t* status, const Geom g) {
  __shared__ float part[NWARPS][R][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;
  const int item = blockIdx.x;
  const int zj = item / g.Hkv, hk = item - zj * g.Hkv;
  const int n = zj / g.J, j = zj - n * g.J;
  const int rows = g.G * g.S;                                    // <= R
  const float c2 = g.sm_scale * GCA_LOG2E;
  float qv[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int e = 0; e < 8; ++e) qv[r][e] = 0.f;
    if (r < rows) {
      const int gi = r / g.S, s = r - gi * g.S;
      const uint4 t = *reinterpret_cast<const uint4*>(q + n * g.qs[0] + j * g.qs[1] + (hk * g.G + gi) * g.qs[2] + s * g.qs[3] + sub * 8);
      const unsigned w4[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { qv[r][2 * e] = bf_lo(w4[e]) * c2; qv[r][2 * e + 1] = bf_hi(w4[e]) * c2; }
    }
  }
  float o[R][8];                                 // this warp's weighted outputs, 8 columns per lane
#pragma unroll
  for (int r = 0; r < R; ++r)
#pragma unroll
    for (int e = 0; e < 8; ++e) o[r][e] = 0.f;
  for (int k = warp; k < g.K; k += NWARPS) {
    const int idx = indices[(long long)zj * g.K + k];
    if (idx < 0) continue;                                       // padding slot (warp-uniform)
    if (idx >= g.C) { if (status && lane == 0) atomicOr(status, GCA_STATUS_BAD_INDEX); continue; }
    const float w = weights[(long long)zj * g.K + k];
    const __nv_bfloat16* kb = kc + n * g.ks[0] + idx * g.ks[1] + hk * g.ks[3] + sub * 8;
    const __nv_bfloat16* vb = vc + n * g.vs[0] + idx * g.vs[1] + hk * g.vs[3] + sub * 8;
    RowState st[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      st[r].m = -INFINITY; st[r].l = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) st[r].acc[e] = 0.f;
    }
    // 16 steps of 4 keys; the loads run four steps ahead of the arithmetic in registers
    uint4 kq[4], vq[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      kq[s] = *reinterpret_cast<const uint4*>(kb + (s * 4 + grp) * g.ks[2]);
      vq[s] = *reinterpret_cast<const uint4*>(vb + (s * 4 + grp) * g.vs[2]);
    }
#pragma unroll 1
    for (int b4 = 0; b4 < 16; b4 += 4) {
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint4 kcur = kq[s], vcur = vq[s];
        if (b4 + 4 < 16) {
          const int key = (b4 + 4 + s) * 4 + grp;
          kq[s] = *reinterpret_cast<const uint4*>(kb + key * g.ks[2]);
          vq[s] = *reinterpret_cast<const uint4*>(vb + key * g.vs[2]);
        }
        const unsigned kw[4] = {kcur.x, kcur.y, kcur.z, kcur.w}, vw[4] = {vcur.x, vcur.y, vcur.z, vcur.w};
        float kf[8], vf[8];
#pragma unroll
        for (int e = 0; e < 4; ++e) { kf[2 * e] = bf_lo(kw[e]); kf[2 * e + 1] = bf_hi(kw[e]); vf[2 * e] = bf_lo(vw[e]); vf[2 * e + 1] = bf_hi(vw[e]); }
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float sc = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) sc = fmaf(qv[r][e], kf[e], sc);
          sc += __shfl_xor_sync(0xffffffffu, sc, 1);
          sc += __shfl_xor_sync(0xffffffffu, sc, 2);
          sc += __shfl_xor_sync(0xffffffffu, sc, 4);
          const float m = fmaxf(st[r].m, sc);
          const float corr = ex2f(st[r].m - m), pr = ex2f(sc - m);
          st[r].l = st[r].l * corr + pr;
#pragma unroll
          for (int e = 0; e < 8; ++e) st[r].acc[e] = fmaf(pr, vf[e], st[r].acc[e] * corr);
          st[r].m = m;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int of = 8; of <= 16; of <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, st[r].m, of), l2 = __shfl_xor_sync(0xffffffffu, st[r].l, of);
        float a2[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) a2[e] = __shfl_xor_sync(0xffffffffu, st[r].acc[e], of);
        merge_state(st[r], m2, l2, a2);
      }
      // softmax over this slot's 64 keys (optionally with the off-by-one term), weighted by w
      float mm = st[r].m, ll = st[r].l;
      if (g.off_by_one > 0.f) {
        const float m1 = fmaxf(mm, 0.f);
        ll = ll * ex2f(mm - m1) + g.off_by_one * ex2f(-m1);
        const float sc1 = ex2f(mm - m1);
#pragma unroll
        for (int e = 0; e < 8; ++e) st[r].acc[e] *= sc1;
      }
      const float f = w / ll;
#pragma unroll
      for (int e = 0; e < 8; ++e) o[r][e] = fmaf(st[r].acc[e], f, o[r][e]);
    }
  }
  if (grp == 0) {
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
      for (int e = 0; e < 8; ++e) part[warp][r][sub * 8 + e] = o[r][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * 64; i += NWARPS * 32) {
    const int r = i >> 6, d = i & 63;
    float t = 0.f;
#pragma unroll
    for (int wv = 0; wv < NWARPS; ++wv) t += part[wv][r][d];
    const int gi = r / g.S, s = r - gi * g.S;
    out[n * g.os[0] + j * g.os[1] + (hk * g.G + gi) * g.os[2] + s * g.os[3] + d] = __float2bfloat16_rn(t);
  }
}

template <int R>
int launch_decode_r(const DecParams& p, int blocks, int sms, cudaStream_t stream) {
  const size_t smem = NWARPS * 2 * TILE_BYTES + 2 * (1 + NWARPS) * R * T * sizeof(float) + 256 + 1024;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(decode_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  decode_kernel<R><<<(unsigned)(blocks < sms ? blocks : sms), NWARPS * 32, smem, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace

// bf16, G*S <= 16 rows.  Returns GCA_ERR_ALGO when the problem is outside that envelope.
int launch_decode(const GcaFwdArgs& a, int sms, cudaStream_t stream) {
  if (a.dtype != GCA_BF16) return GCA_ERR_ALGO;
  DecParams p;
  p.q = (const __nv_bfloat16*)a.q; p.indices = a.indices; p.weights = a.weights;
  p.out = (__nv_bfloat16*)a.out; p.status = a.status;
  Geom& g = p.g;
  g.N = a.N; g.J = a.J; g.Hq = a.Hq; g.Hkv = a.Hkv; g.S = a.S; g.L = a.L; g.D = a.D; g.K = a.K; g.C = a.C;
  g.G = a.Hq / a.Hkv;
  for (int i = 0; i < 4; ++i) { g.qs[i] = a.q_stride[i]; g.os[i] = a.o_stride[i]; g.ks[i] = a.k_stride[i]; g.vs[i] = a.v_stride[i]; }
  g.sm_scale = a.sm_scale; g.off_by_one = a.off_by_one;
  const int rows = g.G * a.S;
  const int blocks = a.N * a.J * a.Hkv;
  // up to four rows: the register-streaming kernel (needs 16-byte aligned 128-byte head rows, which
  // the argument checks of the entry point guarantee for q and the caches)
  bool vec16 = true;                  // every 64-element head row of q and the caches starts on a 16-byte boundary
  for (int i = 0; i < 4; ++i) vec16 = vec16 && a.q_stride[i] % 8 == 0 && a.k_stride[i] % 8 == 0 && a.v_stride[i] % 8 == 0;
  vec16 = vec16 && ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k_cache) | reinterpret_cast<uintptr_t>(a.v_cache)) & 15u) == 0;
  if (rows <= 4 && blocks > 0 && a.D == 64 && a.L == 64 && vec16) {
    auto q = (const __nv_bfloat16*)a.q; auto kc = (const __nv_bfloat16*)a.k_cache; auto vc = (const __nv_bfloat16*)a.v_cache;
    auto out = (__nv_bfloat16*)a.out;
    if (rows <= 1) decode_rows_kernel<1><<<(unsigned)blocks, NWARPS * 32, 0, stream>>>(q, kc, vc, a.indices, a.weights, out, a.status, g);
    else if (rows <= 2) decode_rows_kernel<2><<<(unsigned)blocks, NWARPS * 32, 0, stream>>>(q, kc, vc, a.indices, a.weights, out, a.status, g);
    else decode_rows_kernel<4><<<(unsigned)blocks, NWARPS * 32, 0, stream>>>(q, kc, vc, a.indices, a.weights, out, a.status, g);
    return (int)cudaGetLastError();
  }
  int rc;
  if ((rc = make_tile_map_5d(&p.tm_k, a.k_cache, 64, 64, a.Hkv, a.C, a.N, a.k_stride[2], a.k_stride[3], a.k_stride[1], a.k_stride[0], 1, true))) return rc;
  if ((rc = make_tile_map_5d(&p.tm_v, a.v_cache, 64, 64, a.Hkv, a.C, a.N, a.v_stride[2], a.v_stride[3], a.v_stride[1], a.v_stride[0], 1, false))) return rc;
  if (rows <= 8) return launch_decode_r<8>(p, blocks, sms, stream);
  if (rows <= 16) return launch_decode_r<16>(p, blocks, sms, stream);
  return GCA_ERR_ALGO;
}

}  // namespace gca
