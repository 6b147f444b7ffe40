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

// 64 float32 accumulator values of one row -> bf16 (scaled) -> 128 contiguous bytes in global
// One accumulator row (64 float32 in `acc`) -> scaled bf16 -> 128 contiguous bytes at dst.
// `wide`: dst is 32-byte aligned (checked on the host for the whole tensor).
__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const uint32_t* acc, float scale, bool wide) {
  const float2 sv = make_float2(scale, scale);
  uint32_t w[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) {
    const float2 a = __fmul2_rn(f2(acc[2 * c], acc[2 * c + 1]), sv);
    w[c] = sm100::pack_bf16x2(a.x, a.y);
  }
  if (wide) {
#pragma unroll
    for (int c = 0; c < 4; ++c)
      sm100::st_global_256(reinterpret_cast<uint8_t*>(dst) + 32 * c, w[8 * c], w[8 * c + 1], w[8 * c + 2], w[8 * c + 3],
                    w[8 * c + 4], w[8 * c + 5], w[8 * c + 6], w[8 * c + 7]);
  } else {
#pragma unroll
    for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(dst)[c] = make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
  }
}

// One warp, 32 accumulator rows (lane = row, 64 float32 each in `acc`) -> scaled bf16 -> global
// rows dst_row0 + r * row_stride (elements), 128 contiguous bytes each.  Stored straight from
// the registers every lane of a store instruction would touch a different line; through 4 KB of
// this warp's shared memory (16-byte pieces, XOR-swizzled so that neither the writes nor the
// reads have bank conflicts) every store instruction covers four whole rows instead.
// The staging rows 0-15 start at `stage`, rows 16-31 at `stage + half` (half = 2048: contiguous).
// Rows must be 16-byte aligned.  Ends with all lanes past their reads of the staging memory.
__device__ __forceinline__ void store_rows_staged(uint8_t* stage, int half, __nv_bfloat16* dst_row0, long long row_stride,
                                                  const uint32_t* acc, float scale, int lane) {
  const float2 sv = make_float2(scale, scale);
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const float2 a0 = __fmul2_rn(f2(acc[8 * c + 0], acc[8 * c + 1]), sv), a1 = __fmul2_rn(f2(acc[8 * c + 2], acc[8 * c + 3]), sv);
    const float2 a2 = __fmul2_rn(f2(acc[8 * c + 4], acc[8 * c + 5]), sv), a3 = __fmul2_rn(f2(acc[8 * c + 6], acc[8 * c + 7]), sv);
    *reinterpret_cast<uint4*>(stage + (lane >> 4) * half + (lane & 15) * 128 + ((c ^ (lane & 7)) << 4)) =
        make_uint4(sm100::pack_bf16x2(a0.x, a0.y), sm100::pack_bf16x2(a1.x, a1.y), sm100::pack_bf16x2(a2.x, a2.y),
                   sm100::pack_bf16x2(a3.x, a3.y));
  }
  __syncwarp();
  const int pc = lane & 7, r0 = lane >> 3;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int r = it * 4 + r0;
    const uint4 v = *reinterpret_cast<const uint4*>(stage + (r >> 4) * half + (r & 15) * 128 + ((pc ^ (r & 7)) << 4));
    reinterpret_cast<uint4*>(dst_row0 + r * row_stride)[pc] = v;
  }
  __syncwarp();
}

}  // namespace gca
