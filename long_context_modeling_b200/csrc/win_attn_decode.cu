// Sliding-window causal self-attention with ALiBi for a handful of new positions against the
// cached window (autoregressive decode): what the reference gets from flash-attn's
// flash_attn_with_kvcache(q, k, v, causal=True, window_size=(W, 0), alibi_slopes=m) at
// model/llama.py:684-688.  Per decoded token this reads 2 x (W + 1) x 128 bytes per (sequence, kv
// head) and layer: HBM-bound, no tensor cores.
//
//   s[i, j] = scale * q_i . k_j  -  slope_h * (pos_i - j),   pos_i = T - Sq + i  (bottom-right aligned)
//   visible: pos_i - W <= j <= pos_i;   out_i = softmax_j(s[i, :]) V
//
// One CTA per (sequence, kv head), 8 warps.  A warp load covers FOUR key rows: 8 lanes x 16 bytes
// per 128-byte row, fully coalesced; each 8-lane group owns a stream of keys (j = 4 * step + group)
// with its own online-softmax state (running maximum, sum, 8 output columns per lane), so the loop
// has no cross-lane traffic except the 3-step dot-product reduction inside a group.  Loads run
// PREFETCH steps ahead of the arithmetic (registers), which keeps ~64 KB per SM in flight.  At the
// end the 4 streams of a warp and the 8 warps are merged in a fixed order: the result does not
// depend on scheduling.
//
// RING form (decode of one position per sequence against a FULL window): the window buffer is a
// ring, the step's new K / V row arrives separately and replaces the oldest row.  With a
// device-side count c of rows written so far, the new row goes to physical row p = c mod T, and
// physical row j holds logical position (j - p - 1) mod T.  The CTA that owns the (sequence, kv head)
// block takes row p from the new-row operands, stores it into the ring, and reads every other
// row in place: the window never moves (shifting it costs a full read + write of the window per
// token and layer, more than the attention itself reads).
#include "gca_common.cuh"

namespace gca {

namespace {

constexpr int NWARPS = 8, PREFETCH = 4;

__device__ __forceinline__ float lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct WinParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const float* slopes;        // (Hq) or nullptr
  __nv_bfloat16* out;
  long long qs[3], os[3];     // strides of (n, head, row) in elements; the 64 head dims are contiguous
  long long ks[3], vs[3];     // strides of (n, kv head, position)
  int N, Hq, Hkv, G, Sq, T, window;
  float c2;                   // scale * log2(e)
  // ring form (else nullptr): the new position's rows by strides (n, kv head) and the count of rows written
  const __nv_bfloat16* knew;
  const __nv_bfloat16* vnew;
  const long long* ring;
  long long ns[2];
};

struct State { float m, l, acc[8]; };

__device__ __forceinline__ void merge(State& a, float m2, float l2, const float* acc2) {
  const float m = fmaxf(a.m, m2);
  const float ca = (a.m == -INFINITY) ? 0.f : ex2(a.m - m), cb = (m2 == -INFINITY) ? 0.f : ex2(m2 - m);
  a.l = a.l * ca + l2 * cb;
#pragma unroll
  for (int i = 0; i < 8; ++i) a.acc[i] = a.acc[i] * ca + acc2[i] * cb;
  a.m = m;
}

// Registers are capped so that three CTAs of the one-row kernel share an SM: 32 sequences x 12
// heads = 384 CTAs then run as ONE wave on 148 SMs (with two per SM a second wave of 88 CTAs
// doubled the kernel's duration).
template <int R, bool RING>
__global__ void __launch_bounds__(NWARPS * 32, R == 1 ? 3 : (R == 2 ? 2 : 1))
win_decode_kernel(const WinParams p) {
  __shared__ float part[NWARPS][R][2 + 64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, grp = lane >> 3, sub = lane & 7;
  const int n = blockIdx.x / p.Hkv, hk = blockIdx.x - n * p.Hkv;
  const int rows = p.G * p.Sq;                       // <= R
  // this lane's 8 query values of every row, pre-scaled; the row's ALiBi slope (in log2 units) and position
  float qv[R][8], slope[R];
  int pos[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int gi = r / p.Sq, i = r - gi * p.Sq, h = hk * p.G + gi;
    pos[r] = p.T - p.Sq + i;
    slope[r] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) qv[r][e] = 0.f;
    if (r < rows) {
      slope[r] = p.slopes ? p.slopes[h] * GCA_LOG2E : 0.f;
      const uint4 t = *reinterpret_cast<const uint4*>(p.q + n * p.qs[0] + h * p.qs[1] + i * p.qs[2] + sub * 8);
      const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) { qv[r][2 * e] = lo(w[e]) * p.c2; qv[r][2 * e + 1] = hi(w[e]) * p.c2; }
    }
  }
  State st[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    st[r].m = -INFINITY; st[r].l = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) st[r].acc[e] = 0.f;
  }
  // keys any row can see: [first, T)
  const int first = max(0, p.T - p.Sq - p.window);
  const __nv_bfloat16* kb = p.k + n * p.ks[0] + hk * p.ks[1] + sub * 8;
  const __nv_bfloat16* vb = p.v + n * p.vs[0] + hk * p.vs[1] + sub * 8;
  const int stride = NWARPS * 4;                     // keys per CTA step
  const int base = first + warp * 4;                 // warp-uniform: every lane runs the same steps
  // Ring form: physical row `newest` is the slot of this step's new row.  The loop reads every row from
  // the ring and skips that slot (it still holds the oldest row); the new row is visited afterwards from
  // knew / vnew and stored into the slot.  The count is loaded first but needed only after the first
  // loads have been issued.  The linear form is the ring whose newest row is the last one, nothing skipped.
  const long long written = RING ? *p.ring : 0;
  uint4 kq[PREFETCH], vq[PREFETCH];
#pragma unroll
  for (int s = 0; s < PREFETCH; ++s) {
    const int j = base + grp + s * stride;
    kq[s] = vq[s] = make_uint4(0, 0, 0, 0);
    if (j < p.T) {
      kq[s] = *reinterpret_cast<const uint4*>(kb + j * p.ks[2]);
      vq[s] = *reinterpret_cast<const uint4*>(vb + j * p.vs[2]);
    }
  }
  const int newest = RING ? (int)((unsigned)written % (unsigned)p.T) : p.T - 1;    // the count stays below 2^32 (caller's contract)
  // one key against every row: `ok` = this lane's group counts it; dist[r] = back = pos[r] - (logical position)
  auto visit = [&](const uint4& kc, const uint4& vc, bool ok, int back) {
    const uint32_t kw[4] = {kc.x, kc.y, kc.z, kc.w}, vw[4] = {vc.x, vc.y, vc.z, vc.w};
    float kf[8], vf[8];
#pragma unroll
    for (int e = 0; e < 4; ++e) { kf[2 * e] = lo(kw[e]); kf[2 * e + 1] = hi(kw[e]); vf[2 * e] = lo(vw[e]); vf[2 * e + 1] = hi(vw[e]); }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float sc = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) sc = fmaf(qv[r][e], kf[e], sc);
      sc += __shfl_xor_sync(0xffffffffu, sc, 1);
      sc += __shfl_xor_sync(0xffffffffu, sc, 2);
      sc += __shfl_xor_sync(0xffffffffu, sc, 4);
      // linear form: `back` is the key's position j; ring form: the distance itself (one query position)
      const int dist = RING ? back : pos[r] - back;
      if (r < rows && ok && (RING || (dist >= 0 && dist <= p.window))) {
        sc -= slope[r] * (float)dist;
        const float m = fmaxf(st[r].m, sc);
        const float corr = ex2(st[r].m - m), pr = ex2(sc - m);       // ex2(-inf) = 0 on the first key
        st[r].l = st[r].l * corr + pr;
#pragma unroll
        for (int e = 0; e < 8; ++e) st[r].acc[e] = fmaf(pr, vf[e], st[r].acc[e] * corr);
        st[r].m = m;
      }
    }
  };
  for (int jb = base; jb < p.T; jb += PREFETCH * stride) {
#pragma unroll
    for (int s = 0; s < PREFETCH; ++s) {
      const int j = jb + grp + s * stride;
      const uint4 kc = kq[s], vc = vq[s];
      const int jn = j + PREFETCH * stride;             // refill this register slot
      if (jn < p.T) {
        kq[s] = *reinterpret_cast<const uint4*>(kb + jn * p.ks[2]);
        vq[s] = *reinterpret_cast<const uint4*>(vb + jn * p.vs[2]);
      }
      // every lane of a warp runs the same number of steps (the reduction uses shuffles); keys past the
      // end are masked, and so is the ring's slot of the new row
      if (RING) {
        int dist = newest - j;                          // rows behind the new one, around the ring
        if (dist < 0) dist += p.T;
        visit(kc, vc, j < p.T && dist != 0, dist);
      } else {
        visit(kc, vc, j < p.T, j);
      }
    }
  }
  if (RING && warp == 0) {
    // the new row: attended to at distance 0 (counted by the warp's first stream), then stored over the oldest
    // row -- no thread of this or another CTA reads that row of the ring
    const long long noff = n * p.ns[0] + hk * p.ns[1] + sub * 8;        // this lane's 16 bytes of the new rows
    const uint4 kc = *reinterpret_cast<const uint4*>(p.knew + noff), vc = *reinterpret_cast<const uint4*>(p.vnew + noff);
    visit(kc, vc, grp == 0, 0);
    if (grp == 0) {
      *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(kb) + newest * p.ks[2]) = kc;
      *reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(vb) + newest * p.vs[2]) = vc;
    }
  }
  // merge the 4 key streams of the warp (groups 8 and 16 lanes apart), then the warps
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int of = 8; of <= 16; of <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, st[r].m, of), l2 = __shfl_xor_sync(0xffffffffu, st[r].l, of);
      float a2[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) a2[e] = __shfl_xor_sync(0xffffffffu, st[r].acc[e], of);
      merge(st[r], m2, l2, a2);
    }
    if (grp == 0) {
      if (sub == 0) { part[warp][r][0] = st[r].m; part[warp][r][1] = st[r].l; }
#pragma unroll
      for (int e = 0; e < 8; ++e) part[warp][r][2 + sub * 8 + e] = st[r].acc[e];
    }
  }
  __syncthreads();
  // thread t < rows * 8 finishes 8 output columns of one row
  if (threadIdx.x < rows * 8) {
    const int r = threadIdx.x >> 3, s8 = threadIdx.x & 7;
    State t;
    t.m = -INFINITY; t.l = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) t.acc[e] = 0.f;
    for (int w = 0; w < NWARPS; ++w) merge(t, part[w][r][0], part[w][r][1], &part[w][r][2 + s8 * 8]);
    const float inv = t.l > 0.f ? 1.0f / t.l : 0.f;
    const int gi = r / p.Sq, i = r - gi * p.Sq, h = hk * p.G + gi;
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_bfloat162 b = __floats2bfloat162_rn(t.acc[2 * e] * inv, t.acc[2 * e + 1] * inv);
      o[e] = *reinterpret_cast<const uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(p.out + n * p.os[0] + h * p.os[1] + i * p.os[2] + s8 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The cached window of one decode step, moved on IN PLACE: every (sequence, head) block of T rows drops
// its oldest row and takes the new position's row at the end.  One CTA owns one block of K or V,
// reads it whole into registers (T <= 16 x 256 rows of 128 bytes... 16 bytes per thread and pass),
// synchronises, and writes it back one row down: no second buffer, no concatenation, 2 x T x 128 bytes of
// traffic per block (the torch.cat + copy it replaces moves twice that through slower kernels).
constexpr int SHIFT_THREADS = 256, SHIFT_MAX_VEC = 20;        // 16-byte vectors per thread: blocks of up to 640 rows
__global__ void __launch_bounds__(SHIFT_THREADS)
window_shift_append_kernel(__nv_bfloat16* __restrict__ kwin, __nv_bfloat16* __restrict__ vwin, const __nv_bfloat16* __restrict__ knew,
                           const __nv_bfloat16* __restrict__ vnew, int H, int T, long long ws0, long long ws1, long long ns0,
                           long long ns1) {
  const bool is_v = blockIdx.y != 0;
  const int n = blockIdx.x / H, h = blockIdx.x - n * H;
  uint4* win = reinterpret_cast<uint4*>((is_v ? vwin : kwin) + n * ws0 + h * ws1);     // T rows x 8 vectors, contiguous
  const uint4* fresh = reinterpret_cast<const uint4*>((is_v ? vnew : knew) + n * ns0 + h * ns1);
  const int total = T * 8;                        // vectors in the block
  uint4 r[SHIFT_MAX_VEC];
#pragma unroll
  for (int i = 0; i < SHIFT_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * SHIFT_THREADS + 8;          // the vector one ROW further on
    if (v < total) r[i] = win[v];
    else if (v < total + 8) r[i] = fresh[v - total];            // the last row comes from the new position
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < SHIFT_MAX_VEC; ++i) {
    const int v = threadIdx.x + i * SHIFT_THREADS;
    if (v < total) win[v] = r[i];
  }
}

}  // namespace

int launch_window_shift_append(const WindowAppendArgs& a, cudaStream_t stream) {
  if (a.T * 8 > SHIFT_THREADS * SHIFT_MAX_VEC) return GCA_ERR_SHAPE;
  const dim3 grid((unsigned)(a.N * a.H), 2);
  if (grid.x == 0) return 0;
  window_shift_append_kernel<<<grid, SHIFT_THREADS, 0, stream>>>((__nv_bfloat16*)a.k_window, (__nv_bfloat16*)a.v_window,
                                                                  (const __nv_bfloat16*)a.k_new, (const __nv_bfloat16*)a.v_new, a.H, a.T,
                                                                  a.window_stride[0], a.window_stride[1], a.new_stride[0], a.new_stride[1]);
  return (int)cudaGetLastError();
}

static int launch_window(const WindowDecodeArgs& a, const WindowRingDecodeArgs* ring, cudaStream_t stream) {
  WinParams p;
  p.knew = p.vnew = nullptr; p.ring = nullptr; p.ns[0] = p.ns[1] = 0;
  if (ring) {
    p.knew = (const __nv_bfloat16*)ring->k_new; p.vnew = (const __nv_bfloat16*)ring->v_new;
    p.ring = (const long long*)ring->rows_written; p.ns[0] = ring->new_stride[0]; p.ns[1] = ring->new_stride[1];
  }
  p.q = (const __nv_bfloat16*)a.q; p.k = (const __nv_bfloat16*)a.k; p.v = (const __nv_bfloat16*)a.v;
  p.slopes = a.alibi_slopes; p.out = (__nv_bfloat16*)a.out;
  for (int i = 0; i < 3; ++i) { p.qs[i] = a.q_stride[i]; p.os[i] = a.o_stride[i]; p.ks[i] = a.k_stride[i]; p.vs[i] = a.v_stride[i]; }
  p.N = a.N; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.Sq = a.Sq; p.T = a.T; p.window = a.window;
  p.c2 = a.sm_scale * GCA_LOG2E;
  const int rows = p.G * a.Sq;
  const unsigned grid = (unsigned)(a.N * a.Hkv);
  if (grid == 0) return 0;
  if (ring) {                                      // one new position: G rows per kv head
    if (rows <= 1) win_decode_kernel<1, true><<<grid, NWARPS * 32, 0, stream>>>(p);
    else if (rows <= 2) win_decode_kernel<2, true><<<grid, NWARPS * 32, 0, stream>>>(p);
    else if (rows <= 4) win_decode_kernel<4, true><<<grid, NWARPS * 32, 0, stream>>>(p);
    else return GCA_ERR_SHAPE;
  } else if (rows <= 1) win_decode_kernel<1, false><<<grid, NWARPS * 32, 0, stream>>>(p);
  else if (rows <= 2) win_decode_kernel<2, false><<<grid, NWARPS * 32, 0, stream>>>(p);
  else if (rows <= 4) win_decode_kernel<4, false><<<grid, NWARPS * 32, 0, stream>>>(p);
  else return GCA_ERR_SHAPE;
  return (int)cudaGetLastError();
}

int launch_window_decode(const WindowDecodeArgs& a, cudaStream_t stream) { return launch_window(a, nullptr, stream); }

int launch_window_ring_decode(const WindowRingDecodeArgs& a, cudaStream_t stream) { return launch_window(a.attn, &a, stream); }

}  // namespace gca
