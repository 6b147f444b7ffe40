// Chunk cache append: copies freshly encoded chunks of K and V into a preallocated,
// GPU-resident cache at a chunk position, clearing the landmark (last) row of every chunk
// on the way, and appends the landmark embeddings.  One pass over the new data; replaces
// the concatenate-and-reallocate growth of the reference cache.
#include "gca_common.cuh"

namespace gca {

namespace {

// 16-byte vectors; `row_vecs` vectors per token row, `L` rows per chunk.
__global__ void cache_append_kernel(const uint4* __restrict__ nk, const uint4* __restrict__ nv,
                                    uint4* __restrict__ kc, uint4* __restrict__ vc,
                                    long long new_bs, long long cache_bs, int count, int pos, int L,
                                    int row_vecs, int zero_landmark, long long per_seq) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (i >= per_seq) return;
  const long long chunk_vecs = (long long)L * row_vecs;
  const int c = (int)(i / chunk_vecs);
  const long long r = i % chunk_vecs;
  const int row = (int)(r / row_vecs);
  uint4 a = nk[n * new_bs + i], b = nv[n * new_bs + i];
  if (zero_landmark && row == L - 1) { a = make_uint4(0, 0, 0, 0); b = a; }
  const long long dst = n * cache_bs + (long long)(pos + c) * chunk_vecs + r;
  kc[dst] = a;
  vc[dst] = b;
  (void)count;
}

__global__ void lmk_append_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long src_bs,
                                  long long dst_bs, int pos, int row_vecs, long long per_seq) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const int n = blockIdx.y;
  if (i >= per_seq) return;
  dst[n * dst_bs + (long long)pos * row_vecs + i] = src[n * src_bs + i];
}

}  // namespace

int launch_cache_append(const CacheAppendArgs& a, cudaStream_t stream) {
  const int esize = a.dtype == GCA_BF16 ? 2 : 4;
  const int per_vec = 16 / esize;
  const int row_vecs = a.HD / per_vec;
  const long long per_seq = (long long)a.count * a.L * row_vecs;
  if (per_seq > 0 && a.N > 0) {
    dim3 grid((unsigned)((per_seq + 255) / 256), (unsigned)a.N);
    cache_append_kernel<<<grid, 256, 0, stream>>>((const uint4*)a.new_k, (const uint4*)a.new_v, (uint4*)a.k_cache,
                                                  (uint4*)a.v_cache, a.new_batch_stride / per_vec,
                                                  a.cache_batch_stride / per_vec, a.count, a.pos, a.L, row_vecs,
                                                  a.zero_landmark, per_seq);
    GCA_CUDA_CHECK(cudaGetLastError());
  }
  if (a.new_lmk && a.lmk_cache && a.count > 0 && a.N > 0) {
    const int lrow_vecs = a.Dm / per_vec;
    const long long lper = (long long)a.count * lrow_vecs;
    dim3 grid((unsigned)((lper + 255) / 256), (unsigned)a.N);
    lmk_append_kernel<<<grid, 256, 0, stream>>>((const uint4*)a.new_lmk, (uint4*)a.lmk_cache,
                                                a.new_lmk_batch_stride / per_vec, a.lmk_cache_batch_stride / per_vec,
                                                a.pos, lrow_vecs, lper);
    GCA_CUDA_CHECK(cudaGetLastError());
  }
  return 0;
}

}  // namespace gca
