// Shared declarations for the GCA kernels: argument views, dtype helpers, error checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gca_b200.h"

#define GCA_LOG2E 1.4426950408889634f

#define GCA_CUDA_CHECK(expr)                         \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) return (int)_e;           \
  } while (0)

namespace gca {

// Element-typed load/store that always computes in float.
template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) {
  return __bfloat162float(*p);
}
template <typename T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}

// Problem geometry shared by forward and backward kernels (passed by value).
struct Geom {
  int N, J, Hq, Hkv, S, L, D, K, C, G;
  long long qs[4];   // q   strides n, j, h, s
  long long os[4];   // out / dq strides
  long long ks[4];   // k   strides n, c, l, h
  long long vs[4];   // v   strides n, c, l, h
  float sm_scale;
  float off_by_one;
};

// Inverse retrieval index: for every cache chunk (n, c) the sorted list of (j*K + k)
// entries that retrieved it.  `offsets` has N*C + 1 entries into `sorted_keys`, whose low
// 32 bits hold the entry.
// `unit_tab` lists the chunks in the order the kv-major tensor-core kernel walks them: sequence
// by sequence, and inside a sequence by DECREASING number of retrievers (x = first entry,
// y = one past the last, z = chunk id n*C + c).  CTAs take units round-robin, so every CTA gets
// chunks of every size class; in chunk order the busiest CTA had 8 % more work than the average
// (chunks near the start of a sequence are retrieved by many more queries than late ones).
struct Csr {
  const int* offsets;
  const unsigned long long* sorted_keys;
  const int4* unit_tab;
};

// launch == false: only lay the index out in `workspace` (it was built by an earlier call)
// by_sort: take the radix-sort path even where the single-launch path would do (same bits)
int build_csr(const int32_t* indices, int N, int J, int K, int C, void* workspace, size_t workspace_bytes,
              Csr* out, size_t* used_bytes, cudaStream_t stream, bool launch = true, bool by_sort = false);
size_t csr_workspace_bytes(int N, int J, int K, int C);

// SIMT (CUDA-core, fp32 accumulate) kernels: every dtype, S <= 64, L = D = 64.
int launch_fwd_simt(const GcaFwdArgs& a, cudaStream_t stream);
// stages: GCA_BWD_STAGE_KV and / or GCA_BWD_STAGE_Q
int launch_bwd_simt(const GcaBwdArgs& a, const Csr& csr, float* dw_part, cudaStream_t stream, unsigned stages);

// tcgen05 / TMEM / TMA kernels: bf16, S = L = D = 64.
int launch_fwd_tc(const GcaFwdArgs& a, int sms, cudaStream_t stream);
// rowterm: (N*J, Hq, K, 64) x 16 bytes of scratch the q-major pass fills with the per-row terms of the kv-major pass
int launch_bwd_tc(const GcaBwdArgs& a, const Csr& csr, float* dw_part, uint4* rowterm, int sms, cudaStream_t stream, unsigned stages);

// dw[zj, k] = sum over heads and `parts` partials of dw_part[zj, h, k, part], in a fixed order
int launch_dw_reduce(const float* dw_part, float* dw, int ZJ, int Hq, int K, int parts, cudaStream_t stream);
int bwd_tc_dw_parts();   // partials per (row block, head, slot) that the tensor-core q-major pass writes

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// The entry points run on the device that HOLDS THE BUFFERS, whatever the calling thread's
// current device is (PyTorch calls the backward from an autograd worker thread; a plain C caller
// may never have called cudaSetDevice).  DeviceScope finds the device of a device pointer,
// makes it current for the duration of the call and restores the previous one.
struct DeviceScope {
  int prev = -1, dev = -1, rc = 0;
  explicit DeviceScope(const void* device_ptr);
  ~DeviceScope();
  DeviceScope(const DeviceScope&) = delete;
  DeviceScope& operator=(const DeviceScope&) = delete;
};
// Number of SMs of a device (asked once per device).
int sm_count(int dev);

// Argument rules shared by lmk_score_topk, lmk_topk_workspace_bytes and lmk_score_topk_static.
int check_topk(const LmkTopkArgs* a);

}  // namespace gca
