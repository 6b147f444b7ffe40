// Growable device buffers without copies: a range of virtual addresses is reserved once for the
// largest size a buffer may reach, and physical memory is mapped behind it page by page (2 MB
// granularity) as the buffer grows.  The chunk cache uses it so that appending to a long context
// never re-copies what is already cached (the reference grows its cache with torch.cat on every
// append, model/DRT.py:87-133; a doubling buffer still copies everything at each doubling and
// holds old + new at that moment).  Addresses stay valid while the buffer grows, so views handed
// out earlier, encoded TMA tensor maps and captured CUDA graphs keep working.
//
// Driver entry points are resolved through the runtime (no link against libcuda).  Host code only.
#include <cuda.h>
#include <cuda_runtime.h>

#include "gca_b200.h"
#include "gca_common.cuh"

namespace gca {
namespace {

template <typename Fn>
Fn driver_fn(const char* name) {
  void* f = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
  if (q != cudaDriverEntryPointSuccess) return nullptr;
  return reinterpret_cast<Fn>(f);
}

typedef CUresult (*GranFn)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
typedef CUresult (*ReserveFn)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
typedef CUresult (*AddrFreeFn)(CUdeviceptr, size_t);
typedef CUresult (*CreateFn)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
typedef CUresult (*ReleaseFn)(CUmemGenericAllocationHandle);
typedef CUresult (*MapFn)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
typedef CUresult (*UnmapFn)(CUdeviceptr, size_t);
typedef CUresult (*AccessFn)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);

CUmemAllocationProp device_prop(int device) {
  CUmemAllocationProp prop = {};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  return prop;
}

}  // namespace
}  // namespace gca

extern "C" {

size_t gca_vmem_granularity(int device) {
  static auto fn = gca::driver_fn<gca::GranFn>("cuMemGetAllocationGranularity");
  if (!fn) return 0;
  cudaFree(0);                                   // a context must exist
  const CUmemAllocationProp prop = gca::device_prop(device);
  size_t g = 0;
  return fn(&g, &prop, CU_MEM_ALLOC_GRANULARITY_MINIMUM) == CUDA_SUCCESS ? g : 0;
}

int gca_vmem_reserve(size_t bytes, size_t alignment, void** va_out) {
  static auto fn = gca::driver_fn<gca::ReserveFn>("cuMemAddressReserve");
  if (!va_out) return GCA_ERR_NULL;
  if (!fn) return GCA_ERR_TMA;
  if (bytes == 0) return GCA_ERR_SHAPE;
  cudaFree(0);
  CUdeviceptr p = 0;
  const CUresult r = fn(&p, bytes, alignment, 0, 0);
  if (r != CUDA_SUCCESS) return r == CUDA_ERROR_OUT_OF_MEMORY ? (int)cudaErrorMemoryAllocation : (int)cudaErrorInvalidValue;
  *va_out = reinterpret_cast<void*>(p);
  return 0;
}

// Back [va, va + bytes) with fresh physical memory of `device` (both multiples of the granularity).
int gca_vmem_map(void* va, size_t bytes, int device, unsigned long long* handle_out) {
  static auto create = gca::driver_fn<gca::CreateFn>("cuMemCreate");
  static auto map = gca::driver_fn<gca::MapFn>("cuMemMap");
  static auto access = gca::driver_fn<gca::AccessFn>("cuMemSetAccess");
  static auto release = gca::driver_fn<gca::ReleaseFn>("cuMemRelease");
  if (!va || !handle_out) return GCA_ERR_NULL;
  if (!create || !map || !access || !release) return GCA_ERR_TMA;
  if (bytes == 0) return GCA_ERR_SHAPE;
  const CUmemAllocationProp prop = gca::device_prop(device);
  CUmemGenericAllocationHandle h = 0;
  CUresult r = create(&h, bytes, &prop, 0);
  if (r != CUDA_SUCCESS) return r == CUDA_ERROR_OUT_OF_MEMORY ? (int)cudaErrorMemoryAllocation : (int)cudaErrorInvalidValue;
  r = map(reinterpret_cast<CUdeviceptr>(va), bytes, 0, h, 0);
  if (r != CUDA_SUCCESS) { release(h); return (int)cudaErrorInvalidValue; }
  CUmemAccessDesc desc = {};
  desc.location = prop.location;
  desc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  r = access(reinterpret_cast<CUdeviceptr>(va), bytes, &desc, 1);
  if (r != CUDA_SUCCESS) return (int)cudaErrorInvalidValue;
  *handle_out = (unsigned long long)h;
  return 0;
}

// Undo one gca_vmem_map (the caller has synchronised: nothing may still use the range).
int gca_vmem_unmap(void* va, size_t bytes, unsigned long long handle) {
  static auto unmap = gca::driver_fn<gca::UnmapFn>("cuMemUnmap");
  static auto release = gca::driver_fn<gca::ReleaseFn>("cuMemRelease");
  if (!va) return GCA_ERR_NULL;
  if (!unmap || !release) return GCA_ERR_TMA;
  const CUresult a = unmap(reinterpret_cast<CUdeviceptr>(va), bytes);
  const CUresult b = release((CUmemGenericAllocationHandle)handle);
  return (a == CUDA_SUCCESS && b == CUDA_SUCCESS) ? 0 : (int)cudaErrorInvalidValue;
}

int gca_vmem_free(void* va, size_t bytes) {
  static auto fn = gca::driver_fn<gca::AddrFreeFn>("cuMemAddressFree");
  if (!va) return GCA_ERR_NULL;
  if (!fn) return GCA_ERR_TMA;
  return fn(reinterpret_cast<CUdeviceptr>(va), bytes) == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

}  // extern "C"
