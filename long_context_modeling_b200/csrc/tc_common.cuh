// Small device-side helpers shared by the tensor-core kernels: incremental work-unit
// cursors, ring counters, packed-math row helpers.
#pragma once

#include <stdint.h>

#include "sm100_ptx.cuh"

namespace gca {

// Walk over this CTA's units u = blockIdx.x, +gridDim.x, ... where unit u is the pair
// (outer, inner) = (u / modulus, u % modulus); no division after init.
struct PairCursor {
  int u, outer, inner, douter, dinner, modulus;
  __device__ __forceinline__ void init(int mod) {
    modulus = mod;
    u = blockIdx.x; outer = u / mod; inner = u - outer * mod;
    douter = gridDim.x / mod; dinner = gridDim.x - douter * mod;
  }
  __device__ __forceinline__ void advance() {
    u += gridDim.x; outer += douter; inner += dinner;
    if (inner >= modulus) { inner -= modulus; ++outer; }
  }
  __device__ __forceinline__ int next_outer() const { return outer + douter + ((inner + dinner >= modulus) ? 1 : 0); }
};

// Running stage / phase of a ring of `depth` buffers (no div or mod in the hot loops).
struct Ring {
  uint32_t st, ph;
  int depth;
  __device__ __forceinline__ void init(int d) { st = 0; ph = 0; depth = d; }
  __device__ __forceinline__ void next() { if (++st == (uint32_t)depth) { st = 0; ph ^= 1; } }
};

// Debug profiling (compiled in only with -DGCA_PROFILE): cycles per phase of one lane.
#ifdef GCA_PROFILE
// Event trace of block 0 (debug builds only): buf[64 + event * 256 + slot] = clock at the event.
#define GCA_TRACE_BUF(buf, ev, slot) do { if ((buf) != nullptr && blockIdx.x == 0 && (uint32_t)(slot) < 256u) (buf)[64 + (ev) * 256 + (slot)] = clock64(); } while (0)
#else
#define GCA_TRACE_BUF(buf, ev, slot) do { } while (0)
#endif
#ifdef GCA_PROFILE
struct PhaseTimer {
  long long acc[12];
  long long t;
  bool on;
  __device__ __forceinline__ void init(bool enable) { on = enable; for (int i = 0; i < 12; ++i) acc[i] = 0; if (on) t = clock64(); }
  __device__ __forceinline__ void lap(int i) { if (on) { const long long n = clock64(); acc[i] += n - t; t = n; } }
  __device__ __forceinline__ void dump(long long* dst) { if (on) for (int i = 0; i < 12; ++i) dst[i] = acc[i]; }
};
#else
struct PhaseTimer {
  __device__ __forceinline__ void init(bool) {}
  __device__ __forceinline__ void lap(int) {}
  __device__ __forceinline__ void dump(long long*) {}
};
#endif

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ float2 f2(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }

// 16 float32 accumulator values of one row -> scaled bf16 -> 32 contiguous bytes at dst.
// `wide`: dst is 32-byte aligned (checked on the host for the whole tensor): one 256-bit store,
// a full sector, instead of two 16-byte halves.
__device__ __forceinline__ void store16_bf16(uint8_t* dst, const uint32_t* v, float scale, bool wide) {
  const float2 sv = make_float2(scale, scale);
  uint32_t w[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float2 a = __fmul2_rn(f2(v[2 * i], v[2 * i + 1]), sv);
    w[i] = sm100::pack_bf16x2(a.x, a.y);
  }
  if (wide) sm100::st_global_256(dst, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
  else {
    reinterpret_cast<uint4*>(dst)[0] = make_uint4(w[0], w[1], w[2], w[3]);
    reinterpret_cast<uint4*>(dst)[1] = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

}  // namespace gca
