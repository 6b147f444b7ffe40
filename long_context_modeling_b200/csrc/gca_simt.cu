// CUDA-core GCA kernels with float32 accumulation.  They serve float32 data (the
// accuracy path: tensor cores would round the operands) and any shape the tensor-core
// kernels do not take (S < 64 query rows).  Tiles are 64 keys x 64 dims; one block owns
// one (sequence, query chunk, head) in the q-major kernels and one (sequence, cache
// chunk, kv head) in the kv-major backward kernel, so no atomics are needed and results
// are bit-reproducible.
#include "gca_common.cuh"

namespace gca {

namespace {

constexpr int T = 64;          // tile edge (keys per chunk, head dim, max query rows)
constexpr int LD = T + 1;      // padded leading dimension in shared memory
constexpr int NTHREADS = 256;

// Load a (rows x 64) tile whose rows are `row_stride` elements apart into padded smem.
template <typename E>
__device__ __forceinline__ void load_tile(float* dst, const E* src, long long row_stride, int rows) {
  for (int i = threadIdx.x; i < T * T; i += NTHREADS) {
    int r = i >> 6, c = i & 63;
    dst[r * LD + c] = (r < rows) ? ld_f<E>(src + r * row_stride + c) : 0.f;
  }
}

// acc[a][b] = sum_d A[(4*ty+a)][d] * B[(tx+16*b)][d]      (A, B padded tiles, "NT" product)
__device__ __forceinline__ void mma_nt(const float* A, const float* B, int ty, int tx, float acc[4][4]) {
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
#pragma unroll 8
  for (int d = 0; d < T; ++d) {
    float av[4], bv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = A[(4 * ty + a) * LD + d];
#pragma unroll
    for (int b = 0; b < 4; ++b) bv[b] = B[(tx + 16 * b) * LD + d];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
  }
}

// acc[a][b] += sum_r A[(4*ty+a)][r] * B[r][(tx+16*b)]     ("NN" product)
__device__ __forceinline__ void mma_nn_acc(const float* A, const float* B, int ty, int tx, float acc[4][4]) {
#pragma unroll 8
  for (int r = 0; r < T; ++r) {
    float av[4], bv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = A[(4 * ty + a) * LD + r];
#pragma unroll
    for (int b = 0; b < 4; ++b) bv[b] = B[r * LD + tx + 16 * b];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
  }
}

// acc[a][b] += sum_r A[r][(4*ty+a)] * B[r][(tx+16*b)]     ("TN" product: A used transposed)
__device__ __forceinline__ void mma_tn_acc(const float* A, const float* B, int ty, int tx, float acc[4][4]) {
#pragma unroll 8
  for (int r = 0; r < T; ++r) {
    float av[4], bv[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = A[r * LD + 4 * ty + a];
#pragma unroll
    for (int b = 0; b < 4; ++b) bv[b] = B[r * LD + tx + 16 * b];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
  }
}

// Reduce over the 16 lanes that share a row (lanes with equal ty inside a half warp).
__device__ __forceinline__ float row_max16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float row_sum16(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------
template <typename E>
__global__ void __launch_bounds__(NTHREADS)
fwd_simt_kernel(const E* __restrict__ q, const E* __restrict__ kc, const E* __restrict__ vc,
                const int32_t* __restrict__ indices, const float* __restrict__ weights,
                E* __restrict__ out, float* __restrict__ lse, int32_t* status, Geom g) {
  extern __shared__ float smem[];
  float* sQ = smem;
  float* sK = sQ + T * LD;
  float* sV = sK + T * LD;
  float* sP = sV + T * LD;

  const int zj = blockIdx.x, h = blockIdx.y;
  const int n = zj / g.J, j = zj % g.J, hk = h / g.G;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;

  load_tile<E>(sQ, q + n * g.qs[0] + j * g.qs[1] + h * g.qs[2], g.qs[3], g.S);
  float o[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) o[a][b] = 0.f;
  const float c2 = g.sm_scale * GCA_LOG2E;

  for (int k = 0; k < g.K; ++k) {
    const int idx = indices[(long long)zj * g.K + k];
    const float w = weights[(long long)zj * g.K + k];
    float* lse_row = lse ? lse + (((long long)zj * g.Hq + h) * g.K + k) * g.S : nullptr;
    if (idx < 0 || idx >= g.C) {
      if (idx >= g.C && status && threadIdx.x == 0) atomicOr(status, GCA_STATUS_BAD_INDEX);
      if (lse_row) for (int r = threadIdx.x; r < g.S; r += NTHREADS) lse_row[r] = 0.f;
      continue;
    }
    __syncthreads();
    load_tile<E>(sK, kc + n * g.ks[0] + idx * g.ks[1] + hk * g.ks[3], g.ks[2], T);
    load_tile<E>(sV, vc + n * g.vs[0] + idx * g.vs[1] + hk * g.vs[3], g.vs[2], T);
    __syncthreads();
    float s[4][4];
    mma_nt(sQ, sK, ty, tx, s);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      float m = -INFINITY;
#pragma unroll
      for (int b = 0; b < 4; ++b) { s[a][b] *= c2; m = fmaxf(m, s[a][b]); }
      m = row_max16(m);
      if (g.off_by_one > 0.f) m = fmaxf(m, 0.f);
      float l = 0.f;
#pragma unroll
      for (int b = 0; b < 4; ++b) { s[a][b] = exp2f(s[a][b] - m); l += s[a][b]; }
      l = row_sum16(l);
      if (g.off_by_one > 0.f) l += g.off_by_one * exp2f(-m);
      const int r = 4 * ty + a;
      if (lse_row && tx == 0 && r < g.S) lse_row[r] = m + log2f(l);
      const float f = w / l;
#pragma unroll
      for (int b = 0; b < 4; ++b) sP[r * LD + tx + 16 * b] = s[a][b] * f;
    }
    __syncthreads();
    mma_nn_acc(sP, sV, ty, tx, o);
  }
  E* op = out + n * g.os[0] + j * g.os[1] + h * g.os[2];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = 4 * ty + a;
    if (r < g.S)
#pragma unroll
      for (int b = 0; b < 4; ++b) st_f<E>(op + r * g.os[3] + tx + 16 * b, o[a][b]);
  }
}

// ------------------------------------------------------------------------------------
// backward, shared per-slot math: given Q, dO, K, V tiles in smem and the row LSE,
// produce P*w (sPw) and dS (sdS) tiles in smem and return the per-thread partial of
// sum_rows Di (for dw).  Rows >= S hold zeros.
// ------------------------------------------------------------------------------------
__device__ __forceinline__ float slot_backward_core(const float* sQ, const float* sdO, const float* sK, const float* sV,
                                                    float* sPw, float* sdS, const float* lse_row, float w, float c2,
                                                    int S, int ty, int tx) {
  float s[4][4], dp[4][4];
  mma_nt(sQ, sK, ty, tx, s);
  mma_nt(sdO, sV, ty, tx, dp);
  float di_sum = 0.f;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = 4 * ty + a;
    const bool live = r < S;
    const float m = live ? lse_row[r] : 0.f;
    float di = 0.f;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      s[a][b] = live ? exp2f(s[a][b] * c2 - m) : 0.f;
      di = fmaf(s[a][b], dp[a][b], di);
    }
    di = row_sum16(di);
    if (tx == 0) di_sum += di;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const float pw = s[a][b] * w;
      sPw[r * LD + tx + 16 * b] = pw;
      sdS[r * LD + tx + 16 * b] = pw * (dp[a][b] - di);
    }
  }
  return di_sum;
}

// kv-major: one block per (sequence n, cache chunk c, kv head).  Loops over every
// (query chunk j, slot k) that retrieved the chunk and over the q heads of the group.
template <typename E>
__global__ void __launch_bounds__(NTHREADS)
bwd_kv_simt_kernel(const E* __restrict__ q, const E* __restrict__ kc, const E* __restrict__ vc,
                   const float* __restrict__ weights, const E* __restrict__ dout, const float* __restrict__ lse,
                   E* __restrict__ dk, E* __restrict__ dv, Csr csr, Geom g,
                   long long dos0, long long dos1, long long dos2, long long dos3,
                   long long dks0, long long dks1, long long dks2, long long dks3,
                   long long dvs0, long long dvs1, long long dvs2, long long dvs3) {
  extern __shared__ float smem[];
  float* sK = smem;
  float* sV = sK + T * LD;
  float* sQ = sV + T * LD;
  float* sdO = sQ + T * LD;
  float* sPw = sdO + T * LD;
  float* sdS = sPw + T * LD;

  const int nc = blockIdx.x, hk = blockIdx.y;
  const int n = nc / g.C, c = nc % g.C;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const float c2 = g.sm_scale * GCA_LOG2E;

  float aK[4][4], aV[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) { aK[a][b] = 0.f; aV[a][b] = 0.f; }

  const int beg = csr.offsets[nc], end = csr.offsets[nc + 1];
  if (end > beg) {
    load_tile<E>(sK, kc + n * g.ks[0] + c * g.ks[1] + hk * g.ks[3], g.ks[2], T);
    load_tile<E>(sV, vc + n * g.vs[0] + c * g.vs[1] + hk * g.vs[3], g.vs[2], T);
  }
  for (int e = beg; e < end; ++e) {
    const int entry = (int)(csr.sorted_keys[e] & 0xffffffffull);
    const int j = entry / g.K, k = entry % g.K;
    const long long zj = (long long)n * g.J + j;
    const float w = weights[zj * g.K + k];
    for (int gi = 0; gi < g.G; ++gi) {
      const int h = hk * g.G + gi;
      __syncthreads();
      load_tile<E>(sQ, q + n * g.qs[0] + j * g.qs[1] + h * g.qs[2], g.qs[3], g.S);
      load_tile<E>(sdO, dout + n * dos0 + j * dos1 + h * dos2, dos3, g.S);
      __syncthreads();
      const float* lse_row = lse + ((zj * g.Hq + h) * g.K + k) * g.S;
      slot_backward_core(sQ, sdO, sK, sV, sPw, sdS, lse_row, w, c2, g.S, ty, tx);
      __syncthreads();
      mma_tn_acc(sPw, sdO, ty, tx, aV);   // dV[key][d] += sum_row (w P)[row][key] dO[row][d]
      mma_tn_acc(sdS, sQ, ty, tx, aK);    // dK[key][d] += sum_row dS[row][key] Q[row][d]
    }
  }
  E* dkp = dk + n * dks0 + c * dks1 + hk * dks3;
  E* dvp = dv + n * dvs0 + c * dvs1 + hk * dvs3;
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int r = 4 * ty + a, col = tx + 16 * b;
      st_f<E>(dkp + r * dks2 + col, aK[a][b] * g.sm_scale);
      st_f<E>(dvp + r * dvs2 + col, aV[a][b]);
    }
}

// q-major: one block per (sequence, query chunk, q head): dQ and the per-head part of dw.
template <typename E>
__global__ void __launch_bounds__(NTHREADS)
bwd_q_simt_kernel(const E* __restrict__ q, const E* __restrict__ kc, const E* __restrict__ vc,
                  const int32_t* __restrict__ indices, const float* __restrict__ weights,
                  const E* __restrict__ dout, const float* __restrict__ lse, E* __restrict__ dq,
                  float* __restrict__ dw_part, Geom g,
                  long long dos0, long long dos1, long long dos2, long long dos3) {
  extern __shared__ float smem[];
  float* sQ = smem;
  float* sdO = sQ + T * LD;
  float* sK = sdO + T * LD;
  float* sV = sK + T * LD;
  float* sPw = sV + T * LD;
  float* sdS = sPw + T * LD;
  __shared__ float red[NTHREADS / 32];

  const int zj = blockIdx.x, h = blockIdx.y;
  const int n = zj / g.J, j = zj % g.J, hk = h / g.G;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  const float c2 = g.sm_scale * GCA_LOG2E;

  load_tile<E>(sQ, q + n * g.qs[0] + j * g.qs[1] + h * g.qs[2], g.qs[3], g.S);
  load_tile<E>(sdO, dout + n * dos0 + j * dos1 + h * dos2, dos3, g.S);
  float aQ[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) aQ[a][b] = 0.f;

  for (int k = 0; k < g.K; ++k) {
    const int idx = indices[(long long)zj * g.K + k];
    float* dwp = dw_part + ((long long)zj * g.Hq + h) * g.K + k;
    if (idx < 0 || idx >= g.C) {
      if (threadIdx.x == 0) *dwp = 0.f;
      continue;
    }
    const float w = weights[(long long)zj * g.K + k];
    __syncthreads();
    load_tile<E>(sK, kc + n * g.ks[0] + idx * g.ks[1] + hk * g.ks[3], g.ks[2], T);
    load_tile<E>(sV, vc + n * g.vs[0] + idx * g.vs[1] + hk * g.vs[3], g.vs[2], T);
    __syncthreads();
    const float* lse_row = lse + (((long long)zj * g.Hq + h) * g.K + k) * g.S;
    // dw wants sum_rows <dO, O_k> = sum_rows rowsum(P * dP): use weight 1 for Di, then scale.
    float di = slot_backward_core(sQ, sdO, sK, sV, sPw, sdS, lse_row, 1.0f, c2, g.S, ty, tx);
    // block reduction of di in a fixed order
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) di += __shfl_xor_sync(0xffffffffu, di, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = di;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int i = 0; i < NTHREADS / 32; ++i) t += red[i];
      *dwp = t;
    }
    // dQ[row][d] += w * sum_key dS1[row][key] K[key][d]   (dS1 computed with weight 1)
    float t[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) t[a][b] = 0.f;
    mma_nn_acc(sdS, sK, ty, tx, t);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < 4; ++b) aQ[a][b] = fmaf(w, t[a][b], aQ[a][b]);
  }
  E* dqp = dq + n * g.os[0] + j * g.os[1] + h * g.os[2];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = 4 * ty + a;
    if (r < g.S)
#pragma unroll
      for (int b = 0; b < 4; ++b) st_f<E>(dqp + r * g.os[3] + tx + 16 * b, aQ[a][b] * g.sm_scale);
  }
}

__global__ void dw_reduce_kernel(const float* __restrict__ part, float* __restrict__ dw, int ZJ, int Hq, int K,
                                 int parts) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)ZJ * K) return;
  const long long zj = i / K;
  const int k = (int)(i % K);
  float t = 0.f;
  for (int h = 0; h < Hq; ++h)
    for (int q = 0; q < parts; ++q) t += part[((zj * Hq + h) * K + k) * parts + q];
  dw[i] = t;
}

Geom make_geom(const GcaFwdArgs& a) {
  Geom g;
  g.N = a.N; g.J = a.J; g.Hq = a.Hq; g.Hkv = a.Hkv; g.S = a.S; g.L = a.L; g.D = a.D; g.K = a.K; g.C = a.C;
  g.G = a.Hq / a.Hkv;
  for (int i = 0; i < 4; ++i) { g.qs[i] = a.q_stride[i]; g.os[i] = a.o_stride[i]; g.ks[i] = a.k_stride[i]; g.vs[i] = a.v_stride[i]; }
  g.sm_scale = a.sm_scale; g.off_by_one = a.off_by_one;
  return g;
}

Geom make_geom(const GcaBwdArgs& a) {
  Geom g;
  g.N = a.N; g.J = a.J; g.Hq = a.Hq; g.Hkv = a.Hkv; g.S = a.S; g.L = a.L; g.D = a.D; g.K = a.K; g.C = a.C;
  g.G = a.Hq / a.Hkv;
  for (int i = 0; i < 4; ++i) { g.qs[i] = a.q_stride[i]; g.os[i] = a.dq_stride[i]; g.ks[i] = a.k_stride[i]; g.vs[i] = a.v_stride[i]; }
  g.sm_scale = a.sm_scale; g.off_by_one = a.off_by_one;
  return g;
}

template <typename E>
int fwd_simt_typed(const GcaFwdArgs& a, cudaStream_t stream) {
  const size_t smem = 4 * T * LD * sizeof(float);
  GCA_CUDA_CHECK(cudaFuncSetAttribute(fwd_simt_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)(a.N * a.J), (unsigned)a.Hq);
  fwd_simt_kernel<E><<<grid, NTHREADS, smem, stream>>>((const E*)a.q, (const E*)a.k_cache, (const E*)a.v_cache,
                                                       a.indices, a.weights, (E*)a.out, a.lse, a.status, make_geom(a));
  return (int)cudaGetLastError();
}

template <typename E>
int bwd_simt_typed(const GcaBwdArgs& a, const Csr& csr, float* dw_part, cudaStream_t stream, unsigned stages) {
  const size_t smem = 6 * T * LD * sizeof(float);
  GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_kv_simt_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  GCA_CUDA_CHECK(cudaFuncSetAttribute(bwd_q_simt_kernel<E>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  Geom g = make_geom(a);
  dim3 gkv((unsigned)(a.N * a.C), (unsigned)a.Hkv);
  if (stages & GCA_BWD_STAGE_KV)
  bwd_kv_simt_kernel<E><<<gkv, NTHREADS, smem, stream>>>(
      (const E*)a.q, (const E*)a.k_cache, (const E*)a.v_cache, a.weights, (const E*)a.dout, a.lse,
      (E*)a.dk_cache, (E*)a.dv_cache, csr, g,
      a.do_stride[0], a.do_stride[1], a.do_stride[2], a.do_stride[3],
      a.dk_stride[0], a.dk_stride[1], a.dk_stride[2], a.dk_stride[3],
      a.dv_stride[0], a.dv_stride[1], a.dv_stride[2], a.dv_stride[3]);
  GCA_CUDA_CHECK(cudaGetLastError());
  dim3 gq((unsigned)(a.N * a.J), (unsigned)a.Hq);
  if (stages & GCA_BWD_STAGE_Q)
  bwd_q_simt_kernel<E><<<gq, NTHREADS, smem, stream>>>(
      (const E*)a.q, (const E*)a.k_cache, (const E*)a.v_cache, a.indices, a.weights, (const E*)a.dout, a.lse,
      (E*)a.dq, dw_part, g, a.do_stride[0], a.do_stride[1], a.do_stride[2], a.do_stride[3]);
  return (int)cudaGetLastError();
}

}  // namespace

int launch_fwd_simt(const GcaFwdArgs& a, cudaStream_t stream) {
  if (a.dtype == GCA_BF16) return fwd_simt_typed<__nv_bfloat16>(a, stream);
  if (a.dtype == GCA_F32) return fwd_simt_typed<float>(a, stream);
  return GCA_ERR_DTYPE;
}

int launch_bwd_simt(const GcaBwdArgs& a, const Csr& csr, float* dw_part, cudaStream_t stream, unsigned stages) {
  if (a.dtype == GCA_BF16) return bwd_simt_typed<__nv_bfloat16>(a, csr, dw_part, stream, stages);
  if (a.dtype == GCA_F32) return bwd_simt_typed<float>(a, csr, dw_part, stream, stages);
  return GCA_ERR_DTYPE;
}

int launch_dw_reduce(const float* dw_part, float* dw, int ZJ, int Hq, int K, int parts, cudaStream_t stream) {
  const long long total = (long long)ZJ * K;
  if (total == 0) return 0;
  dw_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(dw_part, dw, ZJ, Hq, K, parts);
  return (int)cudaGetLastError();
}

}  // namespace gca
