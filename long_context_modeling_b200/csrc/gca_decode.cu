// GCA forward for a handful of query rows (autoregressive decode: 1 or 2 rows per
// sequence).  The work is a stream over K retrieved chunks x (K tile + V tile) per
// (sequence, kv head): HBM-bound, no tensor cores.  One block per (n, j, kv head); each
// warp owns whole slots: it stages the slot's 64x64 K and V tiles in shared memory with
// 16-byte coalesced loads, scores the R = G*S query rows against the 64 keys (two keys per
// lane), normalises inside the warp and accumulates its weighted P.V in registers.  The
// per-warp partial outputs are summed in warp order at the end, so the result does not
// depend on scheduling.
#include "gca_common.cuh"

namespace gca {

namespace {

constexpr int T = 64;
constexpr int NWARPS = 8;
constexpr int TILE_BYTES = T * T * 2;      // one bf16 tile

__device__ __forceinline__ float bf_lo(unsigned v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(unsigned v) { return __uint_as_float(v & 0xffff0000u); }

template <int R>
__global__ void __launch_bounds__(NWARPS * 32)
decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ kc,
              const __nv_bfloat16* __restrict__ vc, const int32_t* __restrict__ indices,
              const float* __restrict__ weights, __nv_bfloat16* __restrict__ out, int32_t* status, Geom g) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // per warp: K tile (swizzled 16-byte pieces) then V tile (plain); after the slot loop the
  // same memory holds the per-warp partial outputs.
  unsigned char* my_tiles = smem_raw + (threadIdx.x >> 5) * 2 * TILE_BYTES;
  float* sQ = (float*)(smem_raw + NWARPS * 2 * TILE_BYTES);     // R x 64 floats
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int zj = blockIdx.x / g.Hkv, hk = blockIdx.x % g.Hkv;
  const int n = zj / g.J, j = zj % g.J;
  const int rows = g.G * g.S;                                    // <= R
  const float c2 = g.sm_scale * GCA_LOG2E;

  for (int i = threadIdx.x; i < R * T; i += NWARPS * 32) {
    const int r = i >> 6, d = i & 63;
    float v = 0.f;
    if (r < rows) {
      const int gi = r / g.S, s = r % g.S;
      v = __bfloat162float(q[n * g.qs[0] + j * g.qs[1] + (hk * g.G + gi) * g.qs[2] + s * g.qs[3] + d]);
    }
    sQ[i] = v * c2;
  }
  __syncthreads();

  float o[R][2];
#pragma unroll
  for (int r = 0; r < R; ++r) { o[r][0] = 0.f; o[r][1] = 0.f; }

  for (int k = warp; k < g.K; k += NWARPS) {
    const int idx = indices[(long long)zj * g.K + k];
    if (idx < 0 || idx >= g.C) {
      if (idx >= g.C && status && lane == 0) atomicOr(status, GCA_STATUS_BAD_INDEX);
      continue;
    }
    const float w = weights[(long long)zj * g.K + k];
    const __nv_bfloat16* kp = kc + n * g.ks[0] + idx * g.ks[1] + hk * g.ks[3];
    const __nv_bfloat16* vp = vc + n * g.vs[0] + idx * g.vs[1] + hk * g.vs[3];
    __syncwarp();
    // stage: 512 16-byte pieces per tile, 16 per lane; K pieces are XOR-swizzled by key
#pragma unroll 4
    for (int i = lane; i < 512; i += 32) {
      const int key = i >> 3, pc = i & 7;
      const uint4 kv = *reinterpret_cast<const uint4*>(kp + key * g.ks[2] + pc * 8);
      const uint4 vv = *reinterpret_cast<const uint4*>(vp + key * g.vs[2] + pc * 8);
      *reinterpret_cast<uint4*>(my_tiles + key * 128 + ((pc ^ (key & 7)) << 4)) = kv;
      *reinterpret_cast<uint4*>(my_tiles + TILE_BYTES + key * 128 + (pc << 4)) = vv;
    }
    __syncwarp();
#pragma unroll
    for (int r = 0; r < R; ++r) {
      if (r >= rows) break;
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int pc = 0; pc < 8; ++pc) {
        const uint4 a = *reinterpret_cast<const uint4*>(my_tiles + lane * 128 + ((pc ^ (lane & 7)) << 4));
        const uint4 b = *reinterpret_cast<const uint4*>(my_tiles + (lane + 32) * 128 + ((pc ^ (lane & 7)) << 4));
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
      p0 *= f; p1 *= f;
      float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
      for (int key = 0; key < 32; ++key) {
        const float pa = __shfl_sync(0xffffffffu, p0, key);
        const float pb = __shfl_sync(0xffffffffu, p1, key);
        const unsigned va = *reinterpret_cast<const unsigned*>(my_tiles + TILE_BYTES + key * 128 + lane * 4);
        const unsigned vb = *reinterpret_cast<const unsigned*>(my_tiles + TILE_BYTES + (key + 32) * 128 + lane * 4);
        a0 = fmaf(pa, bf_lo(va), a0); a1 = fmaf(pa, bf_hi(va), a1);
        a0 = fmaf(pb, bf_lo(vb), a0); a1 = fmaf(pb, bf_hi(vb), a1);
      }
      o[r][0] += a0; o[r][1] += a1;
    }
  }
  // cross-warp sum in warp order
  __syncthreads();
  float* part = (float*)smem_raw;                 // NWARPS x R x 64 floats (<= 32 KB)
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
    out[n * g.os[0] + j * g.os[1] + (hk * g.G + gi) * g.os[2] + s * g.os[3] + d] = __float2bfloat16_rn(t);
  }
}

template <int R>
int launch_decode_r(const GcaFwdArgs& a, const Geom& g, cudaStream_t stream) {
  const size_t smem = NWARPS * 2 * TILE_BYTES + R * T * sizeof(float);
  GCA_CUDA_CHECK(cudaFuncSetAttribute(decode_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  decode_kernel<R><<<(unsigned)(a.N * a.J * a.Hkv), NWARPS * 32, smem, stream>>>(
      (const __nv_bfloat16*)a.q, (const __nv_bfloat16*)a.k_cache, (const __nv_bfloat16*)a.v_cache, a.indices,
      a.weights, (__nv_bfloat16*)a.out, a.status, g);
  return (int)cudaGetLastError();
}

}  // namespace

// bf16, G*S <= 16 rows.  Returns GCA_ERR_ALGO when the problem is outside that envelope.
int launch_decode(const GcaFwdArgs& a, cudaStream_t stream) {
  if (a.dtype != GCA_BF16) return GCA_ERR_ALGO;
  Geom g;
  g.N = a.N; g.J = a.J; g.Hq = a.Hq; g.Hkv = a.Hkv; g.S = a.S; g.L = a.L; g.D = a.D; g.K = a.K; g.C = a.C;
  g.G = a.Hq / a.Hkv;
  for (int i = 0; i < 4; ++i) { g.qs[i] = a.q_stride[i]; g.os[i] = a.o_stride[i]; g.ks[i] = a.k_stride[i]; g.vs[i] = a.v_stride[i]; }
  g.sm_scale = a.sm_scale; g.off_by_one = a.off_by_one;
  const int rows = g.G * a.S;
  if (rows <= 1) return launch_decode_r<1>(a, g, stream);
  if (rows <= 2) return launch_decode_r<2>(a, g, stream);
  if (rows <= 4) return launch_decode_r<4>(a, g, stream);
  if (rows <= 8) return launch_decode_r<8>(a, g, stream);
  if (rows <= 16) return launch_decode_r<16>(a, g, stream);
  return GCA_ERR_ALGO;
}

}  // namespace gca
