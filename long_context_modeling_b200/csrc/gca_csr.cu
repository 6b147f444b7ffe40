// Inverse retrieval index for the kv-major backward pass.
//
// For every cache chunk (n, c) the backward needs the list of (query chunk j, slot k)
// pairs that retrieved it, in a fixed order so that float32 accumulation is reproducible.
// Each valid entry becomes the 64-bit key  (n*C + c) << 32 | (j*K + k); a stable radix sort
// on the chunk field gives the lists back to back (two 8-bit passes at N*C = 2048 instead of
// the eight of a full 64-bit sort), and a binary search per chunk finds where each list starts.
// Padding slots (index < 0) and out-of-range indices sort to the end.  Small problems take a
// single-launch counting sort with the same result (csr_small_kernel).
#include <cstdlib>

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
// (first entry, one past the last, chunk id): what the kv-major kernel reads per unit.
__global__ void csr_offsets_kernel(const unsigned long long* __restrict__ sorted, int* __restrict__ offsets,
                                   unsigned* __restrict__ ukeys, int4* __restrict__ uvals,
                                   long long total, long long NC, int C, int cbits, unsigned cmax) {
  const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (c > NC) return;
  const long long lo = csr_lower_bound(sorted, total, (unsigned long long)c << 32);
  offsets[c] = (int)lo;
  if (c == NC) return;
  const unsigned cnt = (unsigned)(csr_lower_bound(sorted, total, (unsigned long long)(c + 1) << 32) - lo);
  ukeys[c] = ((unsigned)(c / C) << cbits) | (cmax - (cnt < cmax ? cnt : cmax));
  uvals[c] = make_int4((int)lo, (int)lo + (int)cnt, (int)c, 0);
}

// ---------------------------------------------------------------------------------------------
// Small problems (C <= 1024 chunks per sequence; the training shapes): the whole index in ONE
// launch, one CTA per sequence, bit-identical to the radix-sort path below, which costs nine
// launches (~85 us, against ~2 ms for the whole backward at the 16K-token shape).
//   1. every warp histograms its own contiguous range of the sequence's J*K entries (shared memory)
//   2. per chunk, an exclusive prefix over the 32 warps; a block scan over the chunks
//   3. every warp walks its range again IN ORDER and places each entry at
//        base(sequence) + start(chunk) + entries of earlier warps + entries earlier in this warp
//      (rank inside a round of 32 by __match_any_sync), i.e. a stable counting sort
//   4. the sequence's chunks sorted by decreasing count (bitonic, shared memory) -> unit table
// base(sequence) = number of valid entries of all earlier sequences, counted by every CTA itself
// (no CTA waits for another).
constexpr int SMALL_C = 1024, SMALL_THREADS = 1024;

__global__ void __launch_bounds__(SMALL_THREADS, 1)
csr_small_kernel(const int32_t* __restrict__ indices, unsigned long long* __restrict__ keys_out, int* __restrict__ offsets,
                 int4* __restrict__ unit_tab, int N, int JK, int C) {
  extern __shared__ int sm[];
  int* hw = sm;                         // [32][C]
  int* start = hw + 32 * C;             // [C + 1]
  int* cnt = start + C + 1;             // [C]
  unsigned* skey = reinterpret_cast<unsigned*>(cnt + C);   // [Cp2]
  int* red = reinterpret_cast<int*>(skey + SMALL_C);       // [33]
  const int n = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int32_t* row = indices + (long long)n * JK;
  for (int i = tid; i < 32 * C; i += SMALL_THREADS) hw[i] = 0;
  // valid entries of the sequences before this one
  int before = 0;
  for (long long i = tid; i < (long long)n * JK; i += SMALL_THREADS) {
    const int v = indices[i];
    before += (v >= 0 && v < C);
  }
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) before += __shfl_xor_sync(0xffffffffu, before, of);
  if (lane == 0) red[warp] = before;
  __syncthreads();
  if (warp == 0) {
    int v = red[lane];
#pragma unroll
    for (int of = 16; of > 0; of >>= 1) v += __shfl_xor_sync(0xffffffffu, v, of);
    if (lane == 0) red[32] = v;
  }
  // 1. per-warp histograms; warp w owns entries [w * per, (w + 1) * per), per a multiple of 32
  const int per = (((JK + 31) / 32) + 31) / 32 * 32;
  const int t0 = warp * per, t1 = min(JK, t0 + per);
  for (int t = t0 + lane; t < t1; t += 32) {
    const int v = row[t];
    if (v >= 0 && v < C) atomicAdd(&hw[warp * C + v], 1);
  }
  __syncthreads();
  const int gbase = red[32];
  // 2. exclusive prefix over the warps per chunk, then over the chunks
  int mine = 0;
  if (tid < C) {
    int run = 0;
    for (int w = 0; w < 32; ++w) { const int v = hw[w * C + tid]; hw[w * C + tid] = run; run += v; }
    cnt[tid] = run;
    mine = run;
  }
  int incl = mine;
#pragma unroll
  for (int of = 1; of < 32; of <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, of); if (lane >= of) incl += v; }
  __syncthreads();                       // red[] is read above by everybody before it is reused
  if (lane == 31) red[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = red[lane], s = v;
#pragma unroll
    for (int of = 1; of < 32; of <<= 1) { const int u = __shfl_up_sync(0xffffffffu, s, of); if (lane >= of) s += u; }
    red[lane] = s - v;                   // exclusive prefix of the warp totals
    if (lane == 31) start[C] = s;        // the sequence's number of valid entries (C <= 1024: all chunks covered)
  }
  __syncthreads();
  if (tid < C) start[tid] = red[warp] + incl - mine;
  __syncthreads();
  // 3. stable placement
  for (int t = t0 + lane; t < t0 + per; t += 32) {      // whole rounds: every lane takes part in the votes
    const int v = t < t1 ? row[t] : -1;
    const bool valid = v >= 0 && v < C;
    const unsigned peers = __match_any_sync(0xffffffffu, valid ? v : -1 - lane);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int pos = 0;
    if (valid) pos = gbase + start[v] + hw[warp * C + v] + rank;
    __syncwarp();
    if (valid) {
      keys_out[pos] = (((unsigned long long)((long long)n * C + v)) << 32) | (unsigned)t;
      if (rank == 0) hw[warp * C + v] += __popc(peers);
    }
    __syncwarp();
  }
  // offsets
  if (tid < C) offsets[(long long)n * C + tid] = gbase + start[tid];
  if (n == N - 1 && tid == 0) offsets[(long long)N * C] = gbase + start[C];
  // 4. walking order of the sequence's chunks: by decreasing count, ties by chunk id
  int cp2 = 1;
  while (cp2 < C) cp2 <<= 1;
  for (int i = tid; i < cp2; i += SMALL_THREADS)
    skey[i] = i < C ? (((unsigned)(JK - cnt[i])) << 10) | (unsigned)i : 0xffffffffu;
  __syncthreads();
  for (int k = 2; k <= cp2; k <<= 1)
    for (int j = k >> 1; j > 0; j >>= 1) {
      for (int i = tid; i < cp2; i += SMALL_THREADS) {
        const int ixj = i ^ j;
        if (ixj > i) {
          const unsigned a = skey[i], b = skey[ixj];
          const bool up = (i & k) == 0;
          if ((a > b) == up) { skey[i] = b; skey[ixj] = a; }
        }
      }
      __syncthreads();
    }
  if (tid < C) {
    const int c = (int)(skey[tid] & 1023u);
    const int beg = gbase + start[c];
    unit_tab[(long long)n * C + tid] = make_int4(beg, beg + cnt[c], n * C + c, 0);
  }
}

size_t small_smem_bytes(int C) { return (size_t)(32 * C + (C + 1) + C + SMALL_C + 33) * 4; }

bool small_path(int N, int JK, int C) {
  return C <= SMALL_C && JK < (1 << 21) && (long long)N * JK <= (1ll << 18);
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
                                  (const int4*)nullptr, (int4*)nullptr, (int)n);
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
         align_up(NC * 4, 256) * 2 + align_up(NC * 16, 256) * 2 + align_up(cub_pairs_temp_bytes(NC), 256);
}

int build_csr(const int32_t* indices, int N, int J, int K, int C, void* workspace, size_t workspace_bytes,
              Csr* out, size_t* used_bytes, cudaStream_t stream, bool launch, bool by_sort) {
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
  int4* uvals_in = (int4*)p;                             p += align_up(NC * 16, 256);
  int4* uvals_out = (int4*)p;                            p += align_up(NC * 16, 256);
  size_t utemp = cub_pairs_temp_bytes(NC);
  void* utemp_ptr = p;
  // a chunk has at most J*K retrievers; the unit key holds (J*K - count) below the sequence number
  const long long cmax = (long long)J * K;
  const int cbits = bits_for(cmax), nbits = bits_for(N);
  if (cbits + nbits > 32) return GCA_ERR_TOO_LARGE;
  if (launch && NC > 0 && total > 0 && !by_sort && small_path(N, J * K, C)) {
    const size_t smem = small_smem_bytes(C);
    GCA_CUDA_CHECK(cudaFuncSetAttribute(csr_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    csr_small_kernel<<<N, SMALL_THREADS, smem, stream>>>(indices, keys_out, offsets, uvals_out, N, J * K, C);
    GCA_CUDA_CHECK(cudaGetLastError());
  } else if (launch) {
    if (total > 0) {
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
    if (NC > 0) {
      csr_offsets_kernel<<<(unsigned)((NC + 1 + 255) / 256), 256, 0, stream>>>(keys_out, offsets, ukeys_in, uvals_in, total,
                                                                               NC, C, cbits, (unsigned)cmax);
      GCA_CUDA_CHECK(cudaGetLastError());
      GCA_CUDA_CHECK(cub::DeviceRadixSort::SortPairs(utemp_ptr, utemp, ukeys_in, ukeys_out, uvals_in, uvals_out, (int)NC, 0,
                                                     cbits + nbits, stream));
    }
  }
  out->offsets = offsets;
  out->sorted_keys = keys_out;
  out->unit_tab = uvals_out;
  *used_bytes = need;
  return 0;
}

}  // namespace gca
