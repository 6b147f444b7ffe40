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
  int M, D, rows_per_seq;   // rows_per_seq = count * 64
  int pos;                  // first chunk position written
  int zero_landmark;
  int tiles_m, tiles_n;     // tiles_n = D / BN
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
  which = r & 1;
  tm = r >> 1;
}

__global__ void __launch_bounds__(NTHREADS, 1)
kv_project_append_kernel(const __grid_constant__ ProjParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total = p.tiles_m * p.tiles_n * 2;
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

}  // namespace

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
  p.tiles_m = (int)((M + BM - 1) / BM); p.tiles_n = a.D / BN;
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
