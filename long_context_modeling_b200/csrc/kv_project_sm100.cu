// Chunk K/V projection fused with the cache append: the two linear maps that turn the chunk
// encoder's output into the chunk cache's K and V (model/DRT.py:770-781 of the reference:
// chunk_k_proj, chunk_v_proj, landmark row cleared) written STRAIGHT into the cache layout at
// the append position (ChunkKVManager.append, model/DRT.py:87-133), and the landmark embeddings
// (the encoder output's last row of every chunk, model/DRT.py:766) copied into the landmark
// cache.  The reference does this as two GEMMs into fresh tensors, two in-place row clears and a
// torch.cat that re-copies the whole cache; here the GEMM's epilogue is the append.
//
//   X  (M = N * count * 64 rows, D columns)  encoder output, bf16, row-major (K-major A operand)
//   Wk, Wv (D x D) bf16 in nn.Linear layout (out, in) = K-major B operand
//   K_cache[n, pos + c, s, :] = X[(n, c, s), :] Wk^T   (zeros for s = 63 when zero_landmark)
//
// tcgen05 GEMM, one CTA per SM, persistent over (row tile of 128, column tile of 256, K|V):
// warp 0 issues the TMA copies of a 4-stage ring (A 128 x 64, B 256 x 64 per stage), warp 1 issues
// 128 x 256 x 16 MMAs into one of two 256-column accumulators in tensor memory, warps 2-5 turn a
// finished accumulator into bf16 rows of the cache while the next tile is being multiplied.
// Every wait is bounded (GCA_STATUS_TIMEOUT on expiry).
//
// The same kernel in LINEAR mode is the projection either side of GCA (model/DRT.py:352-355,385):
//   out[m, :] = row_scale[m] * (x[m, :] W^T) + residual[m, :]
// row_scale = 1 / rms(x) from `row_rms_kernel` turns it into pre-norm RMSNorm + q_proj (the norm's
// gain is folded into W's columns by the caller: RMSNorm(x) W^T = diag(1 / rms) x (W diag(g))^T, so
// the normalised activations are never written), residual makes it o_proj + residual add.
//
// CROSS-ENTROPY mode is the LM head fused with the loss (model/DRT.py:1055-1064, inference /
// evaluation): the 128 x 256 logit tiles stay in tensor memory, the epilogue reduces each row's tile
// to (maximum, sum of exponentials) and picks out the target's logit, and `ce_combine_kernel`
// merges a row's column tiles into  loss = logsumexp - logit[target].  The (rows x 50,265) logits
// -- 13 GB in bf16 at 8 x 16K tokens -- are never written.
#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tc_common.cuh"
#include "tma_host.cuh"

namespace gca {

namespace {

using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OFF_BAR = STAGES * STAGE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int NTHREADS = 6 * 32;
enum Bar { FULL = 0, EMPTY = FULL + STAGES, ACC_FULL = EMPTY + STAGES, ACC_EMPTY = ACC_FULL + 2, NUM_BARS = ACC_EMPTY + 2 };
constexpr uint32_t IDESC = umma_idesc_bf16(BM, BN, 0, 0);

struct ProjParams {
  CUtensorMap tm_x, tm_wk, tm_wv;
  __nv_bfloat16* k_cache;
  __nv_bfloat16* v_cache;
  int32_t* status;
  long long cache_bs;       // elements between sequences in the caches
  int M, D, rows_per_seq;   // D = contraction length; rows_per_seq = count * 64
  int pos;                  // first chunk position written
  int zero_landmark;
  int tiles_m, tiles_n;     // tiles_n = ceil(output columns / BN)
  int nmat;                 // 2: K and V projection with append epilogue; 1: linear mode
  // linear mode
  __nv_bfloat16* out;
  const __nv_bfloat16* residual;      // or nullptr
  const float* row_scale;             // or nullptr
  long long out_stride, res_stride;   // elements between rows
  int ncols;                          // output columns (multiple of 16; any number in cross-entropy mode)
  // cross-entropy mode (linear mode with ce_part != nullptr): the logits never leave tensor memory
  float2* ce_part;                    // (M, tiles_n): running maximum and sum of exp2 of the row's logits in that column tile
  float* ce_target;                   // (M): the target's logit, scaled by log2(e)
  const long long* targets;           // (M) class ids; negative = ignored row
};

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(smem_dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
               : "memory");
}

// tile t of this CTA -> (which matrix, row tile, column tile)
__device__ __forceinline__ void tile_of(const ProjParams& p, int t, int& which, int& tm, int& tn) {
  tn = t % p.tiles_n;
  const int r = t / p.tiles_n;
  if (p.nmat == 2) { which = r & 1; tm = r >> 1; }
  else { which = 0; tm = r; }
}

__global__ void __launch_bounds__(NTHREADS, 1)
kv_project_append_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.tiles_m * p.tiles_n * p.nmat;
  const int ksteps = p.D / BK;
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { mbar_init(&bars[FULL + i], 1); mbar_init(&bars[EMPTY + i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[ACC_FULL + i], 1); mbar_init(&bars[ACC_EMPTY + i], 128); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  if (warp == 0 && lane == 0) { tma_prefetch_desc(&p.tm_x); tma_prefetch_desc(&p.tm_wk); tma_prefetch_desc(&p.tm_wv); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      Ring ring; ring.init(STAGES);
      uint32_t issued = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < total && ok; t += gridDim.x) {
        int which, tm, tn;
        tile_of(p, t, which, tm, tn);
        const CUtensorMap* tw = which ? &p.tm_wv : &p.tm_wk;
        for (int ks = 0; ks < ksteps; ++ks) {
          ok = mbar_wait_bounded(&bars[EMPTY + ring.st], ring.ph ^ 1, abort_flag);
          if (!ok) break;
          uint8_t* dst = smem + ring.st * STAGE_BYTES;
          mbar_arrive_expect_tx(&bars[FULL + ring.st], STAGE_BYTES);
          tma_load_2d(dst, &p.tm_x, &bars[FULL + ring.st], ks * BK, tm * BM);          // rows past M are zero-filled
          tma_load_2d(dst + A_BYTES, tw, &bars[FULL + ring.st], ks * BK, tn * BN);
          ring.next();
          ++issued;
        }
      }
      if (*abort_flag)          // nothing may land in shared memory after the block has gone
        for (uint32_t back = 0; back < (uint32_t)STAGES && back < issued; ++back) {
          const uint32_t g = issued - 1 - back;
          for (int i = 0; i < (1 << 20); ++i)
            if (mbar_try_wait(&bars[FULL + g % STAGES], (g / STAGES) & 1)) break;
        }
    }
  } else if (warp == 1) {
    // all lanes run the issuing code; elect.sync inside the wrappers picks the issuing lane
    Ring ring; ring.init(STAGES);
    bool ok = true;
    uint32_t tcount = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++tcount) {
      const uint32_t ab = tcount & 1;
      ok = mbar_wait_warp(&bars[ACC_EMPTY + ab], ((tcount >> 1) & 1) ^ 1, abort_flag, lane);
      for (int ks = 0; ks < ksteps && ok; ++ks) {
        ok = mbar_wait_warp(&bars[FULL + ring.st], ring.ph, abort_flag, lane);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = umma_desc_sw128(smem_u32(smem + ring.st * STAGE_BYTES));
        const uint64_t db = umma_desc_sw128(smem_u32(smem + ring.st * STAGE_BYTES + A_BYTES));
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
          umma_bf16_ss_elect(tmem_base + ab * BN, da + kk * 2, db + kk * 2, IDESC, (uint32_t)(ks > 0 || kk > 0));
        umma_commit_elect(&bars[EMPTY + ring.st]);
        ring.next();
      }
      if (ok) umma_commit_elect(&bars[ACC_FULL + ab]);
    }
  } else {
    // epilogue: thread = accumulator lane = row of the tile
    const int quad = warp & 3;                           // warps 2..5 -> TMEM lane quarters 2, 3, 0, 1
    const int row_in_tile = quad * 32 + lane;
    const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
    bool ok = true;
    uint32_t tcount = 0;
    for (int t = blockIdx.x; t < total && ok; t += gridDim.x, ++tcount) {
      int which, tm, tn;
      tile_of(p, t, which, tm, tn);
      const uint32_t ab = tcount & 1;
      ok = mbar_wait_bounded(&bars[ACC_FULL + ab], (tcount >> 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, ok)) { ok = false; break; }
      tc_fence_after();
      const long long m = (long long)tm * BM + row_in_tile;
      const bool live = m < p.M;
      if (p.nmat == 1 && p.ce_part) {
        // cross-entropy mode: per row, the maximum and the sum of exponentials of this column
        // tile's logits (base 2, logits scaled by log2 e) and the target's logit if it lies here
        const float sc = ((live && p.row_scale) ? p.row_scale[m] : 1.0f) * GCA_LOG2E;
        const int cols = min(BN, p.ncols - tn * BN);
        const long long tgt = live ? p.targets[m] - (long long)tn * BN : -1;
        float mx = -INFINITY, sum = 0.f;
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(tlane + ab * BN + c0, v);
          tmem_ld_wait();
          float x[16];
          float pm = -INFINITY;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            x[i] = (c0 + i < cols) ? __uint_as_float(v[i]) * sc : -INFINITY;
            pm = fmaxf(pm, x[i]);
          }
          if (tgt >= c0 && tgt < c0 + 16 && tgt < cols) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (tgt == c0 + i) p.ce_target[m] = x[i];
          }
          const float nm = fmaxf(mx, pm);
          float ps = 0.f;
#pragma unroll
          for (int i = 0; i < 16; ++i) ps += ex2_approx(x[i] - nm);
          sum = sum * ex2_approx(mx - nm) + ps;
          mx = nm;
        }
        if (live) p.ce_part[m * p.tiles_n + tn] = make_float2(mx, sum);
        tc_fence_before();
        mbar_arrive(&bars[ACC_EMPTY + ab]);
        continue;
      }
      if (p.nmat == 1) {
        // linear mode: out = row_scale * acc + residual, 16 columns per pass
        const float sc = (live && p.row_scale) ? p.row_scale[m] : 1.0f;
        __nv_bfloat16* orow = p.out + m * p.out_stride + tn * BN;
        const __nv_bfloat16* rrow = p.residual ? p.residual + m * p.res_stride + tn * BN : nullptr;
        const int cols = min(BN, p.ncols - tn * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < cols; c0 += 16) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(tlane + ab * BN + c0, v);
          // the residual's 32 bytes are requested before the accumulator read is waited for
          uint4 r0 = make_uint4(0, 0, 0, 0), r1 = r0;
          if (live && rrow) { r0 = *reinterpret_cast<const uint4*>(rrow + c0); r1 = *reinterpret_cast<const uint4*>(rrow + c0 + 8); }
          tmem_ld_wait();
          if (live) {
            uint32_t w[8];
            if (rrow) {
              const uint32_t rr[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i)
                w[i] = pack_bf16x2(fmaf(__uint_as_float(v[2 * i]), sc, __uint_as_float(rr[i] << 16)),
                                   fmaf(__uint_as_float(v[2 * i + 1]), sc, __uint_as_float(rr[i] & 0xffff0000u)));
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) w[i] = pack_bf16x2(__uint_as_float(v[2 * i]) * sc, __uint_as_float(v[2 * i + 1]) * sc);
            }
            reinterpret_cast<uint4*>(orow + c0)[0] = make_uint4(w[0], w[1], w[2], w[3]);
            reinterpret_cast<uint4*>(orow + c0)[1] = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
        tc_fence_before();
        mbar_arrive(&bars[ACC_EMPTY + ab]);
        continue;
      }
      const int n = live ? (int)(m / p.rows_per_seq) : 0;
      const int r = live ? (int)(m - (long long)n * p.rows_per_seq) : 0;       // (chunk, row) inside the appended block
      const bool zero = p.zero_landmark && (r & 63) == 63;
      __nv_bfloat16* dst = (which ? p.v_cache : p.k_cache) + n * p.cache_bs + ((long long)p.pos * 64 + r) * p.D + tn * BN;
      // one small loop body (16 columns: TMEM -> bf16 -> one 32-byte store), 16 passes
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tlane + ab * BN + c0, v);
        tmem_ld_wait();
        if (zero) {
#pragma unroll
          for (int i = 0; i < 16; ++i) v[i] = 0u;
        }
        if (live) store16_bf16(reinterpret_cast<uint8_t*>(dst + c0), v, 1.0f, true);
      }
      tc_fence_before();
      mbar_arrive(&bars[ACC_EMPTY + ab]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

// 2-D bf16 matrix (rows x cols, row stride in elements), boxes of (64 columns x box_rows rows), 128-byte swizzle.
int make_matrix_map(CUtensorMap* map, const void* base, long long rows, long long cols, long long row_stride, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return GCA_ERR_TMA;
  if (row_stride % 8 != 0) return GCA_ERR_STRIDE;
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)row_stride * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : GCA_ERR_TMA;
}

__global__ void lmk_rows_kernel(const uint4* __restrict__ x, uint4* __restrict__ lmk, long long lmk_bs, int pos, int count,
                                int row_vecs, long long total) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int v = (int)(i % row_vecs);
  const long long cn = i / row_vecs;                      // n * count + c
  const int c = (int)(cn % count);
  const long long n = cn / count;
  lmk[n * lmk_bs + (long long)(pos + c) * row_vecs + v] = x[(cn * 64 + 63) * row_vecs + v];
}

// row_scale[m] = rsqrt(mean(x[m, :]^2) + eps): one warp per row, 16-byte loads.
__global__ void row_rms_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ row_scale, long long M, int D,
                               long long stride, float eps) {
  const long long m = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const int lane = threadIdx.x & 31;
  const uint4* row = reinterpret_cast<const uint4*>(x + m * stride);
  float acc = 0.f;
  for (int i = lane; i < D / 8; i += 32) {
    const uint4 v = row[i];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = __uint_as_float(w[j] << 16), b = __uint_as_float(w[j] & 0xffff0000u);
      acc = fmaf(a, a, acc); acc = fmaf(b, b, acc);
    }
  }
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
  if (lane == 0) row_scale[m] = rsqrtf(acc / (float)D + eps);
}

// out[m, c] = silu(gu[m, c]) * gu[m, I + c]: the activation between one gate|up product and down_proj
// (the reference's fused SwiGLU, model/llama.py:290-300).  One thread per 8 columns, 16-byte accesses.
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out, long long M, int I,
                                long long in_stride, long long out_stride) {
  const int per_row = I / 8;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= M * per_row) return;
  const long long m = t / per_row;
  const int c = (int)(t - m * per_row) * 8;
  const uint4 g = *reinterpret_cast<const uint4*>(gu + m * in_stride + c);
  const uint4 u = *reinterpret_cast<const uint4*>(gu + m * in_stride + I + c);
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float g0 = __uint_as_float(gw[j] << 16), g1 = __uint_as_float(gw[j] & 0xffff0000u);
    const float u0 = __uint_as_float(uw[j] << 16), u1 = __uint_as_float(uw[j] & 0xffff0000u);
    const __nv_bfloat162 b = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
    o[j] = *reinterpret_cast<const uint32_t*>(&b);
  }
  *reinterpret_cast<uint4*>(out + m * out_stride + c) = make_uint4(o[0], o[1], o[2], o[3]);
}

// loss[m] = ln(sum_j exp(logit_j)) - logit_target from the per-tile partials (base 2 inside); ignored rows: 0.
__global__ void ce_combine_kernel(const float2* __restrict__ part, const float* __restrict__ tlogit, const long long* __restrict__ targets,
                                  float* __restrict__ loss, float* __restrict__ lse_out, long long M, int tiles) {
  const long long m = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (m >= M) return;
  const int lane = threadIdx.x & 31;
  float mx = -INFINITY, sum = 0.f;
  for (int t = lane; t < tiles; t += 32) {
    const float2 v = part[m * tiles + t];
    const float nm = fmaxf(mx, v.x);
    sum = sum * (mx == -INFINITY ? 0.f : exp2f(mx - nm)) + v.y * (v.x == -INFINITY ? 0.f : exp2f(v.x - nm));
    mx = nm;
  }
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, mx, of), os = __shfl_xor_sync(0xffffffffu, sum, of);
    const float nm = fmaxf(mx, om);
    sum = sum * (mx == -INFINITY ? 0.f : exp2f(mx - nm)) + os * (om == -INFINITY ? 0.f : exp2f(om - nm));
    mx = nm;
  }
  if (lane == 0) {
    const float lse2 = mx + log2f(sum);                        // base-2 log-sum-exp of the scaled logits
    const float ln2 = 0.6931471805599453f;
    if (lse_out) lse_out[m] = lse2 * ln2;
    loss[m] = targets[m] >= 0 ? (lse2 - tlogit[m]) * ln2 : 0.f;
  }
}

}  // namespace

int launch_linear_ce(const LinearCeArgs& a, int sms, cudaStream_t stream) {
  ProjParams p;
  int rc;
  if ((rc = make_matrix_map(&p.tm_x, a.x, a.M, a.K, a.x_stride, BM)) || (rc = make_matrix_map(&p.tm_wk, a.w, a.N, a.K, a.w_stride, BN)))
    return rc;
  p.tm_wv = p.tm_wk;
  p.k_cache = p.v_cache = nullptr; p.status = a.status; p.cache_bs = 0;
  p.M = (int)a.M; p.D = a.K; p.rows_per_seq = 1; p.pos = 0; p.zero_landmark = 0;
  p.tiles_m = (int)((a.M + BM - 1) / BM); p.tiles_n = (a.N + BN - 1) / BN; p.nmat = 1;
  p.out = nullptr; p.residual = nullptr; p.row_scale = a.row_scale; p.out_stride = p.res_stride = 0; p.ncols = a.N;
  // workspace: partials (M, tiles_n) float2, then the target logits (M) float
  p.ce_part = reinterpret_cast<float2*>(a.workspace);
  p.ce_target = reinterpret_cast<float*>(p.ce_part + a.M * p.tiles_n);
  p.targets = reinterpret_cast<const long long*>(a.targets);
  const long long total = (long long)p.tiles_m * p.tiles_n;
  if (total >= (1ll << 31) || a.M >= (1ll << 31)) return GCA_ERR_TOO_LARGE;
  if (total == 0) return 0;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(kv_project_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  kv_project_append_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  GCA_CUDA_CHECK(cudaGetLastError());
  const int warps = 8;
  ce_combine_kernel<<<(unsigned)((a.M + warps - 1) / warps), warps * 32, 0, stream>>>(p.ce_part, p.ce_target, p.targets, a.loss, a.lse, a.M,
                                                                                    p.tiles_n);
  return (int)cudaGetLastError();
}

int launch_row_rms(const RowRmsArgs& a, cudaStream_t stream) {
  if (a.M == 0) return 0;
  const int warps = 8;
  row_rms_kernel<<<(unsigned)((a.M + warps - 1) / warps), warps * 32, 0, stream>>>(
      (const __nv_bfloat16*)a.x, a.row_scale, a.M, a.D, a.x_stride, a.eps);
  return (int)cudaGetLastError();
}

int launch_silu_mul(const void* gu, void* out, long long M, int I, long long in_stride, long long out_stride, cudaStream_t stream) {
  const long long threads = M * (I / 8);
  if (threads == 0) return 0;
  silu_mul_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, M, I, in_stride,
                                                                            out_stride);
  return (int)cudaGetLastError();
}

int launch_linear(const LinearArgs& a, int sms, cudaStream_t stream) {
  ProjParams p;
  int rc;
  if ((rc = make_matrix_map(&p.tm_x, a.x, a.M, a.K, a.x_stride, BM)) || (rc = make_matrix_map(&p.tm_wk, a.w, a.N, a.K, a.w_stride, BN)))
    return rc;
  p.tm_wv = p.tm_wk;
  p.k_cache = p.v_cache = nullptr; p.status = a.status; p.cache_bs = 0;
  p.M = (int)a.M; p.D = a.K; p.rows_per_seq = 1; p.pos = 0; p.zero_landmark = 0;
  p.tiles_m = (int)((a.M + BM - 1) / BM); p.tiles_n = (a.N + BN - 1) / BN; p.nmat = 1;
  p.out = (__nv_bfloat16*)a.out; p.residual = (const __nv_bfloat16*)a.residual; p.row_scale = a.row_scale;
  p.out_stride = a.out_stride; p.res_stride = a.residual_stride; p.ncols = a.N;
  p.ce_part = nullptr; p.ce_target = nullptr; p.targets = nullptr;
  const long long total = (long long)p.tiles_m * p.tiles_n;
  if (total >= (1ll << 31) || a.M >= (1ll << 31)) return GCA_ERR_TOO_LARGE;
  if (total == 0) return 0;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(kv_project_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  kv_project_append_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  GCA_CUDA_CHECK(cudaGetLastError());
  return 0;
}

int launch_kv_project_append(const KvProjectArgs& a, int sms, cudaStream_t stream) {
  ProjParams p;
  const long long M = (long long)a.N * a.count * 64;
  int rc;
  if ((rc = make_matrix_map(&p.tm_x, a.x, M, a.D, a.D, BM)) || (rc = make_matrix_map(&p.tm_wk, a.wk, a.D, a.D, a.D, BN)) ||
      (rc = make_matrix_map(&p.tm_wv, a.wv, a.D, a.D, a.D, BN)))
    return rc;
  p.k_cache = (__nv_bfloat16*)a.k_cache; p.v_cache = (__nv_bfloat16*)a.v_cache; p.status = a.status;
  p.cache_bs = a.cache_batch_stride; p.M = (int)M; p.D = a.D; p.rows_per_seq = a.count * 64; p.pos = a.pos;
  p.zero_landmark = a.zero_landmark;
  p.tiles_m = (int)((M + BM - 1) / BM); p.tiles_n = a.D / BN; p.nmat = 2;
  p.out = nullptr; p.residual = nullptr; p.row_scale = nullptr; p.out_stride = p.res_stride = 0; p.ncols = a.D;
  p.ce_part = nullptr; p.ce_target = nullptr; p.targets = nullptr;
  const long long total = (long long)p.tiles_m * p.tiles_n * 2;
  if (total >= (1ll << 31)) return GCA_ERR_TOO_LARGE;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(kv_project_append_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(total < sms ? total : sms);
  kv_project_append_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  GCA_CUDA_CHECK(cudaGetLastError());
  if (a.lmk_cache) {
    const int row_vecs = a.D / 8;
    const long long tot = (long long)a.N * a.count * row_vecs;
    lmk_rows_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, stream>>>((const uint4*)a.x, (uint4*)a.lmk_cache,
                                                                      a.lmk_cache_batch_stride / 8, a.pos, a.count, row_vecs, tot);
    GCA_CUDA_CHECK(cudaGetLastError());
  }
  return 0;
}

}  // namespace gca
