// Inverse retrieval index for the kv-major backward pass.
//
// For every cache chunk (n, c) the backward needs the list of (query chunk j, slot k)
// pairs that retrieved it, in a fixed order so that float32 accumulation is reproducible.
// Each valid entry becomes the 64-bit key  (n*C + c) << 32 | (j*K + k); a stable radix sort
// on the chunk field gives the lists back to back (two 8-bit passes at N*C = 2048 instead of
// the eight of a full 64-bit sort), and a binary search per chunk finds where each list starts.  Padding slots (index < 0) and out-of-range indices sort to the end.
#include <cub/device/device_radix_sort.cuh>

#include "gca_common.cuh"

namespace gca {

namespace {

__global__ void csr_keys_kernel(const int32_t* __restrict__ indices, unsigned long long* __restrict__ keys,
                                int N, int JK, int C) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)N * JK) return;
  const int n = (int)(i / JK);
  const int t = (int)(i % JK);
  const int idx = indices[i];
  keys[i] = (idx < 0 || idx >= C) ? ~0ull
                                  : (((unsigned long long)((long long)n * C + idx)) << 32) | (unsigned)t;
}

__device__ __forceinline__ long long csr_lower_bound(const unsigned long long* __restrict__ sorted, long long total,
                                                     unsigned long long target) {
  long long lo = 0, hi = total;
  while (lo < hi) {
    const long long mid = (lo + hi) >> 1;
    if (sorted[mid] < target) lo = mid + 1; else hi = mid;
  }
  return lo;
}

// offsets[c] = first sorted key of chunk c (or the end).  The same thread also emits the chunk's
// entry of the kv-major walking order: key = sequence << cbits | (cmax - count), so that an
// ascending sort lists a sequence's chunks by decreasing number of retrievers; value =
// chunk id << 32 | first entry.
__global__ void csr_offsets_kernel(const unsigned long long* __restrict__ sorted, int* __restrict__ offsets,
                                   unsigned* __restrict__ ukeys, unsigned long long* __restrict__ uvals,
                                   long long total, long long NC, int C, int cbits, unsigned cmax) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (c > NC) return;
  const long long lo = csr_lower_bound(sorted, total, (unsigned long long)c << 32);
  offsets[c] = (int)lo;
  if (c == NC) return;
  const unsigned cnt = (unsigned)(csr_lower_bound(sorted, total, (unsigned long long)(c + 1) << 32) - lo);
  ukeys[c] = ((unsigned)(c / C) << cbits) | (cmax - (cnt < cmax ? cnt : cmax));
  uvals[c] = ((unsigned long long)c << 32) | (unsigned long long)lo;
}

size_t cub_temp_bytes(long long total) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortKeys(nullptr, bytes, (const unsigned long long*)nullptr,
                                 (unsigned long long*)nullptr, (int)total);
  return bytes;
}

size_t cub_pairs_temp_bytes(long long n) {
  size_t bytes = 0;
  cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const unsigned*)nullptr, (unsigned*)nullptr,
                                  (const unsigned long long*)nullptr, (unsigned long long*)nullptr, (int)n);
  return bytes;
}

int bits_for(long long v) {       // smallest b with 2^b > v
  int b = 0;
  while ((1ll << b) <= v) ++b;
  return b;
}

}  // namespace

size_t csr_workspace_bytes(int N, int J, int K, int C) {
  const long long total = (long long)N * J * K;
  const long long NC = (long long)N * C;
  return align_up(total * 8, 256) * 2 + align_up((NC + 1) * 4, 256) + align_up(cub_temp_bytes(total), 256) +
         align_up(NC * 4, 256) * 2 + align_up(NC * 8, 256) * 2 + align_up(cub_pairs_temp_bytes(NC), 256);
}

int build_csr(const int32_t* indices, int N, int J, int K, int C, void* workspace, size_t workspace_bytes,
              Csr* out, size_t* used_bytes, cudaStream_t stream, bool launch) {
  const long long total = (long long)N * J * K;
  const long long NC = (long long)N * C;
  if (total >= (1ll << 31) || NC >= (1ll << 31)) return GCA_ERR_TOO_LARGE;
  const size_t need = csr_workspace_bytes(N, J, K, C);
  if (!workspace || workspace_bytes < need) return GCA_ERR_WORKSPACE;
  char* p = (char*)workspace;
  unsigned long long* keys_in = (unsigned long long*)p;  p += align_up(total * 8, 256);
  unsigned long long* keys_out = (unsigned long long*)p; p += align_up(total * 8, 256);
  int* offsets = (int*)p;                                p += align_up((NC + 1) * 4, 256);
  size_t temp = cub_temp_bytes(total);
  void* temp_ptr = p;                                    p += align_up(temp, 256);
  unsigned* ukeys_in = (unsigned*)p;                     p += align_up(NC * 4, 256);
  unsigned* ukeys_out = (unsigned*)p;                    p += align_up(NC * 4, 256);
  unsigned long long* uvals_in = (unsigned long long*)p; p += align_up(NC * 8, 256);
  unsigned long long* uvals_out = (unsigned long long*)p; p += align_up(NC * 8, 256);
  size_t utemp = cub_pairs_temp_bytes(NC);
  void* utemp_ptr = p;
  if (launch && total > 0) {
    csr_keys_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(indices, keys_in, N, J * K, C);
    GCA_CUDA_CHECK(cudaGetLastError());
    // The keys are generated in increasing (j*K + k) order inside a sequence, and the radix sort
    // is stable, so sorting on the chunk field alone is a full sort.  Valid chunk ids are < N*C
    // <= 2^b; the all-ones key of an invalid entry has bit b set and sorts behind them.
    int b = 0;
    while ((1ll << b) < NC) ++b;
    const int end_bit = 32 + b + 1 > 64 ? 64 : 32 + b + 1;
    GCA_CUDA_CHECK(cub::DeviceRadixSort::SortKeys(temp_ptr, temp, keys_in, keys_out, (int)total, 32, end_bit, stream));
  }
  // a chunk has at most J*K retrievers; the key holds (J*K - count) below the sequence number
  const long long cmax = (long long)J * K;
  const int cbits = bits_for(cmax), nbits = bits_for(N);
  if (cbits + nbits > 32) return GCA_ERR_TOO_LARGE;
  if (launch && NC > 0) {
    csr_offsets_kernel<<<(unsigned)((NC + 1 + 255) / 256), 256, 0, stream>>>(keys_out, offsets, ukeys_in, uvals_in, total, NC,
                                                                             C, cbits, (unsigned)cmax);
    GCA_CUDA_CHECK(cudaGetLastError());
    GCA_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(utemp_ptr, utemp, ukeys_in, ukeys_out, uvals_in, uvals_out, (int)NC, 0,
                                                   cbits + nbits, stream));
  }
  out->offsets = offsets;
  out->sorted_keys = keys_out;
  out->unit_keys = ukeys_out;
  out->unit_vals = uvals_out;
  out->unit_cmax = (unsigned)cmax;
  out->unit_cmask = (1u << cbits) - 1u;
  *used_bytes = need;
  return 0;
}

}  // namespace gca
