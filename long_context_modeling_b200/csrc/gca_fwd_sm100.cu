// GCA forward on the 5th-generation tensor cores (tcgen05 + TMEM), bf16, S = L = D = 64.
//
// Work unit: one (sequence n, query chunk j, PAIR of q heads A, B).  The two heads are
// stacked along M so every MMA is a full 128-row instruction:
//
//   S  = [Q_A; Q_B] [K_A; K_B]^T   M=128, N=128, K=64: the diagonal 64x64 blocks are the two
//                                  heads' scores (rows 0-63 x cols 0-63, rows 64-127 x cols
//                                  64-127); the off-diagonal blocks are computed and ignored
//   O += [P_A; P_B] [V_A | V_B]    same shape, V as MN-major B operand spanning both heads
//
// Issuing one tcgen05.mma costs the issuing thread ~70-100 cycles whatever its shape
// (measured), and a 64x64x16 instruction is only 32 cycles of tensor work, so with these tiny
// tiles the instruction count -- not the FLOP count -- is what must be minimised: stacking
// the heads halves it, and the discarded off-diagonal half of the result is free.  With GQA,
// when both q heads share one kv head, N is 64 and nothing is discarded.
//
// Per retrieved slot k (padding slots are skipped):  S -> one thread per row computes
// P = (w_k / l) * exp2(S c - m) in bf16 (no running rescale: a slot's softmax spans exactly
// one key tile) -> O accumulates over all K slots in ONE TMEM tile (fused weighted merge).
// K_k / V_k tiles for both heads arrive with ONE TMA copy each, straight from the chunk
// cache with the retrieved chunk index as a tensor coordinate (no gathered copy exists).
//
// CTA = 16 warps.
//   warps 0-11  three softmax warpgroups (thread = TMEM lane = row); a group reads S from one of
//               two accumulators and writes P into its own 32 columns of tensor memory, so one
//               group's chain S -> TMEM read -> exp2 -> P -> PV overlaps the other two groups'
//   warp  12    walks the unit list, publishes one DESCRIPTOR per unit in shared memory (valid
//               slots, retrieved indices, weights, output / lse offsets, and which group takes
//               which slot), issues the TMA copies of Q and K
//   warp  13    TMA producer for V (separate ring; K is released as soon as S is done)
//   warp  14    issues the S MMAs;  warp 15 the PV MMAs (one O accumulator, slots in order, so
//               the result does not depend on timing)
// Warps 0-11 and 13-15 only follow descriptors: the unit bookkeeping (index rows, divisions,
// 64-bit offsets, padding slots) is ~100 rarely executed, branchy instructions that cost a
// warp ~10 cycles each, and it used to sit on every warpgroup's critical path once per unit.
// A warp can issue one tcgen05.mma per ~100 cycles when it runs converged with warp-uniform
// operands and only the instruction itself is predicated on elect.sync (~150 inside a
// divergent `if (lane == 0)` region), so the issuing warps run all lanes.  Ring stages are
// released by tcgen05.commit straight onto the producers' barriers.  CTAs are persistent and
// walk the units in (n, j, head pair) order so that concurrently running CTAs touch the cache
// of few sequences (L2 reuse of chunks retrieved many times).  Every mbarrier wait is bounded;
// on expiry the CTA flags GCA_STATUS_TIMEOUT, drains its copies and unwinds.
#include <cstdlib>

#include "gca_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace gca {

namespace {

using namespace sm100;

constexpr int TILE_BYTES = 64 * 64 * 2;
constexpr int PAIR_BYTES = 2 * TILE_BYTES;
constexpr int NWG = 3;                      // softmax warpgroups
constexpr int NSB = 2;                      // S accumulators in tensor memory: slot g uses g % 2
constexpr int NK = 6, NV = 6;               // K / V ring stages
constexpr int ND = 4;                       // unit descriptors in flight
#ifndef GCA_FWD_SKIP
#define GCA_FWD_SKIP 4
#endif
#ifndef GCA_OUT_COLS
#define GCA_OUT_COLS 16
#endif
constexpr int OUT_COLS = GCA_OUT_COLS;      // columns per pass of the output loop (16 or 32)
constexpr int FWD_SKIP = GCA_FWD_SKIP;      // slots at the start of a unit that the previous unit's output writer sits out (even)
constexpr int NTHREADS = (4 * NWG + 4) * 32;
constexpr int KPROD_WARP = 4 * NWG, VPROD_WARP = KPROD_WARP + 1, SMMA_WARP = KPROD_WARP + 2;   // last warp: PV issuer
// Tensor memory: S0 | S1 | O (128 columns each) | P0 P1 P2 (32 columns each).  P -- the bf16
// probabilities, one row per lane, two values per column -- is the A operand of the PV product
// straight from tensor memory: it never goes through shared memory, whose 128 bytes per clock
// (operand reads of the MMAs + TMA writes) are the kernel's tightest resource.
constexpr int TMEM_COLS = 512;
constexpr int TMEM_O = NSB * 128, TMEM_P = TMEM_O + 128;

// What the other roles need to know about a unit.  The warp that issues the Q / K copies walks
// the unit list, reads the retrieved indices and weights, does all the index and address
// arithmetic ONCE and publishes the result here; the other 15 warps only follow descriptors.
// (Each role used to walk the list itself: ~100 rarely executed, branchy instructions per unit
// that are never in the instruction cache, ~2,000 cycles per unit on every warpgroup's critical path.)
struct UnitDesc {
  uint32_t mask;            // valid slots of the unit
  uint32_t flags;           // DESC_*; bits 4-5: the warpgroup that writes the unit's output
  int32_t n, hk0;           // sequence and first kv head: tensor coordinates of the V copies
  long long lse_off;        // element offset of (unit, head A, slot 0, row 0) in lse
  long long out_off;        // element offset of (unit, head A, row 0) in out
  uint32_t own[3];          // the slots of each warpgroup
  uint32_t g0;              // running number of the unit's first slot (traces)
};
constexpr uint32_t DESC_END = 1, DESC_TWO = 2, DESC_SHARE = 4, DESC_EPI_SHIFT = 4;
static_assert(sizeof(UnitDesc) == 48, "descriptor header");
// Per slot one byte: bits 0-2 = slot number modulo 6 (ring stage / barrier of the slot; bit 0 is
// also the S accumulator), bits 3-4 = the slot's warpgroup.
constexpr int DESC_HDR = 48, DESC_ONE = DESC_HDR + 128 + 128 + 32;

constexpr int OFF_Q = 0;                              // [2 bufs][A B]
constexpr int OFF_K = OFF_Q + 2 * PAIR_BYTES;         // [NK][A B]
constexpr int OFF_V = OFF_K + NK * PAIR_BYTES;        // [NV][A B]
constexpr int OFF_BAR = OFF_V + NV * PAIR_BYTES;
constexpr int OFF_DESC = OFF_BAR + 512;               // [ND] headers | [ND][32] indices | [ND][32] weights | [ND][32] slot bytes
constexpr int DESC_BYTES = ND * DESC_ONE;
static_assert(NK == 6 && NV == 6, "slot bytes carry the slot number modulo 6");
constexpr int SMEM_BYTES = OFF_DESC + DESC_BYTES + 1024;   // + alignment slack

// Barriers.
//   DESC_FULL[d]   descriptor d is written (1 arrival);  DESC_EMPTY[d]: its 15 readers are done
//   K_FULL[stage]  the slot's K tile has landed (producer's expect_tx arrival + bytes) AND the S
//                  accumulator the slot will use has been read by the group that had it two slots
//                  earlier (its 4 warps arrive here); the S issuer's only wait
//   S_FULL[group]  S of the group's next slot is complete (commit)
//   K_EMPTY[stage] same commit, for the K producer
//   V_FULL[stage]  the V tile has landed AND the slot's group has written P; the PV issuer's only wait
//   P_EMPTY[group] PV of the group's latest slot is complete (commit): its P region may be rewritten
//   V_EMPTY[stage] same commit, for the V producer
//   O_FULL[group]  the unit whose last slot the group had is accumulated; O_EMPTY: O has been read
// A barrier that belongs to a group completes one phase per slot of that group, and the next
// phase cannot complete before the group has acted on this one, so parity is never ambiguous
// whatever the assignment of slots to groups is.
enum Bar { Q_FULL = 0, Q_EMPTY = 2, K_FULL = 4, K_EMPTY = K_FULL + NK, V_FULL = K_EMPTY + NK, V_EMPTY = V_FULL + NV,
           S_FULL = V_EMPTY + NV, P_EMPTY = S_FULL + NWG, O_FULL = P_EMPTY + NWG, O_EMPTY = O_FULL + NWG,
           DESC_FULL = O_EMPTY + 1, DESC_EMPTY = DESC_FULL + ND, NUM_BARS = DESC_EMPTY + ND };
constexpr int DESC_READERS = 4 * NWG + 3;   // softmax warps, the two MMA issuers, the V producer
static_assert(NUM_BARS * 8 + 16 <= 512, "barrier block");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");

struct FwdTcParams {
  CUtensorMap tm_q, tm_k2, tm_v2, tm_k1, tm_v1;   // *2: both heads of a pair per copy, *1: one head
  const int32_t* indices;
  const float* weights;
  __nv_bfloat16* out;
  float* lse;
  int32_t* status;
  long long* prof;          // optional cycle counters of block 0 (debug), or nullptr
  long long os[4];
  int units;
  int N, J, Hq, Hkv, G, K, C, HP;
  int pair;                 // 1: a unit is a pair of q heads; 0: a single head (GCA_ALGO_TC_UNPAIRED)
  int dbg;                  // profile builds only: bit mask of work to skip (timing experiments)
  int wide_store;           // every output row is 32-byte aligned: 256-bit stores
  float c2;
  float off_by_one;
};

// Debug tracing (compiled in only with -DGCA_PROFILE).
#ifdef GCA_PROFILE
// event trace of block 0: prof[64 + event * 256 + slot] = clock of that event for that slot
#define GCA_TRACE(ev, slot) do { if (p.prof != nullptr && blockIdx.x == 0 && (slot) < 256u) p.prof[64 + (ev) * 256 + (slot)] = clock64(); } while (0)
#else
#define GCA_TRACE(ev, slot) do { } while (0)
#endif

// Timing experiments (compiled in only with -DGCA_DBGKNOBS): skip parts of the work.
#ifdef GCA_DBGKNOBS
#define GCA_DBG(bit) ((p.dbg >> (bit)) & 1)
#else
#define GCA_DBG(bit) 0
#endif

// Incremental walk over this CTA's units u = blockIdx.x, +gridDim.x, ...: unit u is
// (zj, hp) = (u / HP, u % HP); no division after the first step.
struct UnitCursor {
  int u, zj, hp, dzj, dhp;
  __device__ __forceinline__ void init(const FwdTcParams& p) {
    u = blockIdx.x; zj = u / p.HP; hp = u - zj * p.HP;
    dzj = gridDim.x / p.HP; dhp = gridDim.x - dzj * p.HP;
  }
  __device__ __forceinline__ void advance(const FwdTcParams& p) {
    u += gridDim.x; zj += dzj; hp += dhp;
    if (hp >= p.HP) { hp -= p.HP; ++zj; }
  }
  __device__ __forceinline__ int next_zj(const FwdTcParams& p) const { return zj + dzj + ((hp + dhp >= p.HP) ? 1 : 0); }
};
struct UnitInfo { int h0, hk0; bool two, share; };
__device__ __forceinline__ UnitInfo unit_info(const FwdTcParams& p, int hp) {
  UnitInfo t;
  t.h0 = p.pair ? 2 * hp : hp;
  t.two = p.pair && (t.h0 + 1) < p.Hq;
  if (p.G == 1) { t.hk0 = t.h0; t.share = false; }
  else { t.hk0 = t.h0 / p.G; t.share = t.two && ((t.h0 + 1) / p.G == t.hk0); }
  return t;
}
// Lane-parallel read of one row of retrieved indices; every role prefetches the next row.
__device__ __forceinline__ int load_index_row(const FwdTcParams& p, int u, int zj, int lane) {
  if (u >= p.units || lane >= p.K) return -1;
  return p.indices[(long long)zj * p.K + lane];
}
__device__ __forceinline__ unsigned valid_mask(const FwdTcParams& p, int idx) {
  return __ballot_sync(0xffffffffu, idx >= 0 && idx < p.C);
}

// Running slot counters of a ring / double buffer (no div or mod in the slot loops).
struct Ring {
  uint32_t st, ph;
  int depth;
  __device__ __forceinline__ void init(int d) { st = 0; ph = 0; depth = d; }
  __device__ __forceinline__ void next() { if (++st == (uint32_t)depth) { st = 0; ph ^= 1; } }
};

__device__ __forceinline__ UnitDesc* desc_hdr(uint8_t* smem) { return reinterpret_cast<UnitDesc*>(smem + OFF_DESC); }
__device__ __forceinline__ int* desc_idx(uint8_t* smem) { return reinterpret_cast<int*>(smem + OFF_DESC + ND * DESC_HDR); }
__device__ __forceinline__ float* desc_w(uint8_t* smem) { return reinterpret_cast<float*>(smem + OFF_DESC + ND * (DESC_HDR + 128)); }
__device__ __forceinline__ uint8_t* desc_slot(uint8_t* smem) { return smem + OFF_DESC + ND * (DESC_HDR + 256); }

// Bounded wait (one lane) for the copies of a ring that may still be in flight: no bulk copy
// may land in shared memory after the CTA has exited.
__device__ __forceinline__ void drain_ring(uint64_t* bars, int full0, uint32_t issued, int depth) {
  for (uint32_t back = 0; back < (uint32_t)depth && back < issued; ++back) {
    const uint32_t g = issued - 1 - back;
    for (int i = 0; i < (1 << 20); ++i)
      if (mbar_try_wait(&bars[full0 + g % depth], (g / depth) & 1)) break;
  }
}

// ----------------------------------------------------------------------------- Q / K producer
// Walks this CTA's units, publishes one descriptor per unit that has valid slots, issues the
// unit's Q copy and one K copy per slot.  Everything a unit needs that no slot will write is
// also done here (rare: the first K chunks of a sequence): zero output rows of a unit without
// valid slots, zero lse of padding slots, the bad-index status bit.
__device__ void kproducer_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane) {
  UnitDesc* hdr = desc_hdr(smem);
  int* didx = desc_idx(smem);
  float* dw = desc_w(smem);
  uint8_t* dslot = desc_slot(smem);
  UnitCursor c;
  c.init(p);
  Ring ring; ring.init(NK);
  Ring dr; dr.init(ND);
  uint32_t un = 0, issued = 0;
  uint32_t g0 = 0, g0m6 = 0;             // running number of the unit's first slot, and modulo 6
  int L = NWG - 1;                       // the group that wrote the previous unit's output
  bool ok = true;
  const unsigned full = (p.K >= 32) ? 0xffffffffu : ((1u << p.K) - 1u);
  int next_idx = load_index_row(p, c.u, c.zj, lane);
  float next_w = (c.u < p.units && lane < p.K) ? p.weights[(long long)c.zj * p.K + lane] : 0.f;
  for (; c.u < p.units && ok; c.advance(p)) {
    const int my_idx = next_idx;
    const float my_w = next_w;
    {
      const int nzj = c.next_zj(p);
      next_idx = load_index_row(p, c.u + gridDim.x, nzj, lane);
      next_w = (c.u + gridDim.x < p.units && lane < p.K) ? p.weights[(long long)nzj * p.K + lane] : 0.f;
    }
    const unsigned mask = valid_mask(p, my_idx);
    const UnitInfo t = unit_info(p, c.hp);
    const int n = c.zj / p.J, j = c.zj - n * p.J;
    const long long lse_off = ((long long)c.zj * p.Hq + t.h0) * p.K * 64;
    const long long out_off = n * p.os[0] + j * p.os[1] + t.h0 * p.os[2];
    if (__any_sync(0xffffffffu, my_idx >= p.C) && p.status && lane == 0) atomicOr(p.status, GCA_STATUS_BAD_INDEX);
    if (mask != full) {
      const int rows = t.two ? 128 : 64;                       // rows of the unit: head A, then head B
      if (p.lse)
        for (int k = 0; k < p.K; ++k)
          if (!((mask >> k) & 1))
            for (int i = lane; i < rows; i += 32) p.lse[lse_off + ((long long)(i >> 6) * p.K + k) * 64 + (i & 63)] = 0.f;
      if (mask == 0) {
        for (int i = lane; i < rows * 8; i += 32) {
          const int r = i >> 3;
          reinterpret_cast<uint4*>(p.out + out_off + (r >> 6) * p.os[2] + (r & 63) * p.os[3])[i & 7] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
    }
    // publish the descriptor
    ok = mbar_wait_warp(&bars[DESC_EMPTY + dr.st], dr.ph ^ 1, abort_flag, lane);
    if (!ok) break;
    didx[dr.st * 32 + lane] = my_idx;
    dw[dr.st * 32 + lane] = my_w;
    // Which warpgroup takes which slot (lane k works out slot k).  The group that has a unit's
    // last slot also writes the unit's output (wait for the last PV, read O, store: ~3,000
    // cycles); with plain rotation its next slot -- and, O being accumulated in slot order, every
    // slot behind it -- would wait for that.  So the first four slots of the next unit alternate
    // between the other two groups and the writer rejoins at the fifth: L = writer of the
    // previous unit, A, B the other two:  slot 0 1 2 3 4 5 6 7 8 ...  ->  A B A B L A B L A ...
    // No group ever has two consecutive slots.
    const bool valid = (mask >> lane) & 1u;
    const int r = __popc(mask & ((1u << lane) - 1u));          // the slot's number inside the unit
    int wgk;
    {
#ifdef GCA_FWD_ROUND_ROBIN
      const int x = (int)(g0 % 3u) + r;
      wgk = x - 3 * ((x * 86) >> 8);
#else
      const int A = L + 1 == NWG ? 0 : L + 1, B = A + 1 == NWG ? 0 : A + 1;
      const int y = r - FWD_SKIP, y3 = y - 3 * ((y * 86) >> 8);   // (r - FWD_SKIP) % 3 for FWD_SKIP <= r < 32
      wgk = r < FWD_SKIP ? ((r & 1) ? B : A) : (y3 == 0 ? L : (y3 == 1 ? A : B));
#endif
    }
    const int xs = (int)g0m6 + r, s6 = xs - 6 * ((xs * 43) >> 8);   // (g0 + r) % 6
    if (valid) dslot[dr.st * 32 + lane] = (uint8_t)(s6 | (wgk << 3));
    const uint32_t own0 = __ballot_sync(0xffffffffu, valid && wgk == 0);
    const uint32_t own1 = __ballot_sync(0xffffffffu, valid && wgk == 1);
    const uint32_t own2 = __ballot_sync(0xffffffffu, valid && wgk == 2);
    const int nv = __popc(mask);
    L = __shfl_sync(0xffffffffu, wgk, 31 - __clz(mask));       // the group of the unit's last slot
    if (lane == 0) {
      UnitDesc h;
      h.mask = mask;
      h.flags = (t.two ? DESC_TWO : 0u) | (t.share ? DESC_SHARE : 0u) | ((uint32_t)L << DESC_EPI_SHIFT);
      h.n = n; h.hk0 = t.hk0; h.lse_off = lse_off; h.out_off = out_off;
      h.own[0] = own0; h.own[1] = own1; h.own[2] = own2; h.g0 = g0;
      hdr[dr.st] = h;
    }
    g0 += nv;
    g0m6 += nv; g0m6 -= 6 * ((g0m6 * 43) >> 8);
    mbar_arrive_warp(&bars[DESC_FULL + dr.st], lane);
    const uint32_t ds = dr.st;
    dr.next();
    if (lane == 0) {
      const uint32_t qb = un & 1;
      ok = mbar_wait_bounded(&bars[Q_EMPTY + qb], ((un >> 1) & 1) ^ 1, abort_flag);
      if (ok) {
        mbar_arrive_expect_tx(&bars[Q_FULL + qb], PAIR_BYTES);
        tma_load_5d(smem + OFF_Q + qb * PAIR_BYTES, &p.tm_q, &bars[Q_FULL + qb], 0, 0, t.h0, j, n);
        const CUtensorMap* tm = t.share ? &p.tm_k1 : &p.tm_k2;
        const uint32_t bytes = t.share ? TILE_BYTES : PAIR_BYTES;
        for (unsigned m = mask; m; m &= m - 1) {
#ifdef GCA_TEST_WITHHOLD_K
          // Test build only: the CTA's first K tile is never requested, so the S issuer's bounded
          // wait for it must expire.  This lane idles (bounded) until some role has given up, then
          // unwinds like after any expired wait: nothing was issued that could still be in flight
          // except the Q copy, which the drain below waits for.
          if (issued == 0) {
            for (uint32_t spin = 0; spin < 64u * GCA_WAIT_LIMIT && !*abort_flag; ++spin) __nanosleep(32);
            ok = false;
            break;
          }
#endif
          ok = mbar_wait_bounded(&bars[K_EMPTY + ring.st], ring.ph ^ 1, abort_flag);
          if (!ok) break;
          mbar_arrive_expect_tx(&bars[K_FULL + ring.st], bytes);
          tma_load_5d(smem + OFF_K + ring.st * PAIR_BYTES, tm, &bars[K_FULL + ring.st], 0, 0, t.hk0,
                      didx[ds * 32 + __ffs(m) - 1], n);
          ring.next();
          ++issued;
        }
      }
    }
    ++un;
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
  }
  // end of work
  if (ok && mbar_wait_warp(&bars[DESC_EMPTY + dr.st], dr.ph ^ 1, abort_flag, lane)) {
    if (lane == 0) { hdr[dr.st].mask = 0; hdr[dr.st].flags = DESC_END; }
    mbar_arrive_warp(&bars[DESC_FULL + dr.st], lane);
  }
  if (lane == 0 && *abort_flag) {
    drain_ring(bars, K_FULL, issued, NK);
    drain_ring(bars, Q_FULL, un, 2);
  }
}

// ----------------------------------------------------------------------------- V producer
__device__ void vproducer_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane) {
  const UnitDesc* hdr = desc_hdr(smem);
  const int* didx = desc_idx(smem);
  Ring ring; ring.init(NV);
  Ring dr; dr.init(ND);
  uint32_t issued = 0;
  bool ok = true;
  while (ok) {
    ok = mbar_wait_warp(&bars[DESC_FULL + dr.st], dr.ph, abort_flag, lane);
    if (!ok) break;
    const UnitDesc h = hdr[dr.st];
    if (h.flags & DESC_END) break;
    if (lane == 0) {
      const bool share = (h.flags & DESC_SHARE) != 0;
      const CUtensorMap* tm = share ? &p.tm_v1 : &p.tm_v2;
      const uint32_t bytes = share ? TILE_BYTES : PAIR_BYTES;
      for (unsigned m = h.mask; m; m &= m - 1) {
        ok = mbar_wait_bounded(&bars[V_EMPTY + ring.st], ring.ph ^ 1, abort_flag);
        if (!ok) break;
        mbar_arrive_expect_tx(&bars[V_FULL + ring.st], bytes);
        tma_load_5d(smem + OFF_V + ring.st * PAIR_BYTES, tm, &bars[V_FULL + ring.st], 0, 0, h.hk0,
                    didx[dr.st * 32 + __ffs(m) - 1], h.n);
        ring.next();
        ++issued;
      }
    }
    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    mbar_arrive_warp(&bars[DESC_EMPTY + dr.st], lane);
    dr.next();
  }
  if (lane == 0 && *abort_flag) drain_ring(bars, V_FULL, issued, NV);
}

// ----------------------------------------------------------------------------- MMA issuers
// mode 0: S = Q K^T into accumulator g % 2;  mode 1: O += P V with P (the slot's group's region
// of tensor memory) as the A operand.  All 32 lanes run this code; elect.sync inside the MMA /
// commit wrappers picks the issuing lane.
template <int MODE>
__device__ void issuer_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int lane,
                            uint32_t tmem_base) {
  constexpr uint32_t PAIR16 = PAIR_BYTES >> 4;
  constexpr uint32_t FULL = MODE == 0 ? K_FULL : V_FULL, EMPTY = MODE == 0 ? K_EMPTY : V_EMPTY;
  const UnitDesc* hdr = desc_hdr(smem);
  const uint64_t dQ = umma_desc_sw128(smem_u32(smem + OFF_Q));
  const uint64_t dB = MODE == 0 ? umma_desc_sw128(smem_u32(smem + OFF_K))
                                : umma_desc_sw128_mn_blocks(smem_u32(smem + OFF_V), TILE_BYTES);
  const uint8_t* dslot = desc_slot(smem);
  Ring dr; dr.init(ND);
  uint32_t un = 0, g = 0;                     // units; running slot number
  uint32_t ph6 = 0;                           // (g / 6) & 1
  bool ok = true;
  while (ok) {
    ok = mbar_wait_warp(&bars[DESC_FULL + dr.st], dr.ph, abort_flag, lane);
    if (!ok) break;
    const uint32_t mask = hdr[dr.st].mask, flags = hdr[dr.st].flags;
    if (flags & DESC_END) break;
    const uint32_t ub = un & 1;
    const uint32_t idesc = umma_idesc_bf16(128, (flags & DESC_SHARE) ? 64 : 128, 0, MODE);
    if (MODE == 0) ok = mbar_wait_warp(&bars[Q_FULL + ub], (un >> 1) & 1, abort_flag, lane);
    else ok = mbar_wait_warp(&bars[O_EMPTY], (un & 1) ^ 1, abort_flag, lane);
    ++un;
    for (uint32_t m = mask; m && ok; m &= m - 1, ++g) {
      const uint32_t info = dslot[dr.st * 32 + __ffs(m) - 1];
      const uint32_t s6 = info & 7u, w = info >> 3;                    // slot number mod 6; the slot's warpgroup
      ok = mbar_wait_warp(&bars[FULL + s6], ph6, abort_flag, lane);    // tile landed and S accumulator free / P written
      if (lane == 0) GCA_TRACE(2 + 3 * MODE, g);
      if (!ok) break;
      tc_fence_after();
      const uint64_t b = dB + s6 * PAIR16;
      const bool last = (m & (m - 1)) == 0;
      if (MODE == 0) {
        const uint64_t a = dQ + ub * PAIR16;
        const uint32_t dt = tmem_base + (s6 & 1u) * 128;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_bf16_ss_elect(dt, a + kk * 2, b + kk * 2, idesc, (uint32_t)(kk > 0));
        umma_commit_elect(&bars[S_FULL + w]);
      } else {
        const uint32_t at = tmem_base + TMEM_P + w * 32;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ts_elect(tmem_base + TMEM_O, at + kk * 8, b + kk * 128, idesc, (uint32_t)(m != mask || kk > 0));
        umma_commit_elect(&bars[P_EMPTY + w]);
      }
      umma_commit_elect(&bars[EMPTY + s6]);                            // the ring stage is free
      if (last) umma_commit_elect(&bars[MODE == 0 ? Q_EMPTY + ub : O_FULL + w]);
      if (lane == 0) GCA_TRACE(4 + 3 * MODE, g);
      if (s6 == 5) ph6 ^= 1;
    }
    mbar_arrive_warp(&bars[DESC_EMPTY + dr.st], lane);
    dr.next();
  }
}

// ----------------------------------------------------------------------------- softmax + epilogue
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ void softmax_role(const FwdTcParams& p, uint8_t* smem, uint64_t* bars, volatile int* abort_flag, int wg,
                             int quad, int lane, uint32_t tmem_base) {
  const int tile = quad >> 1;                       // TMEM lanes 0-63: head A, 64-127: head B
  const int row = (quad & 1) * 32 + lane;           // query row inside the head
  const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
  const bool elected = quad == 0 && lane == 0;
  const uint32_t tP = tlane + TMEM_P + (uint32_t)wg * 32;   // this warpgroup's P region of tensor memory
  const UnitDesc* hdr = desc_hdr(smem);
  const float* dw = desc_w(smem);
  // this thread's row inside a unit's output / lse block
  __nv_bfloat16* const out_t = p.out + tile * p.os[2] + row * p.os[3];
  const long long lse_t = (long long)tile * p.K * 64 + row;
  const bool wide_store = p.wide_store != 0;
  const uint8_t* dslot = desc_slot(smem);
  Ring dr; dr.init(ND);
  uint32_t own = 0, epi = 0;                        // own slots / outputs done
  bool ok = true;
  // slots 0 and 1 find their S accumulators untouched: groups 1 and 2 stand in for the readers of
  // "slots -2 and -1" (a slot's reader arrives on the K barrier of the slot two later)
  if (wg >= 1) mbar_arrive_warp(&bars[K_FULL + (wg - 1)], lane);

  while (ok) {
    ok = mbar_wait_warp(&bars[DESC_FULL + dr.st], dr.ph, abort_flag, lane);
    if (!ok) break;
    const uint32_t flags = hdr[dr.st].flags;
    if (flags & DESC_END) break;
    const uint32_t mine = hdr[dr.st].own[wg];        // this group's slots
    const long long lse_off = hdr[dr.st].lse_off, out_off = hdr[dr.st].out_off;
    const float my_w = dw[dr.st * 32 + lane];        // lane k: weight and slot byte of slot k
    const uint32_t my_info = dslot[dr.st * 32 + lane];
#ifdef GCA_PROFILE
    const uint32_t umask = hdr[dr.st].mask, g0 = hdr[dr.st].g0;
#endif
    mbar_arrive_warp(&bars[DESC_EMPTY + dr.st], lane);
    dr.next();
    const bool live = tile == 0 || (flags & DESC_TWO);
    const uint32_t coff = (flags & DESC_SHARE) ? 0u : (uint32_t)tile * 64u;
    float* lse_base = p.lse ? p.lse + lse_off + lse_t : nullptr;
    __nv_bfloat16* orow = out_t + out_off;
    for (unsigned m = mine; m; m &= m - 1) {
      const int k = __ffs(m) - 1;
      const float wk = __shfl_sync(0xffffffffu, my_w, k);
      const uint32_t vs = __shfl_sync(0xffffffffu, my_info, k) & 7u;   // slot number mod 6: V barrier, S accumulator
      const uint32_t kn = vs + 2 >= 6 ? vs - 4 : vs + 2;               // K barrier of the slot two later
#ifdef GCA_PROFILE
      const uint32_t gt = g0 + __popc(umask & ((1u << k) - 1u));
#endif
      if (elected) GCA_TRACE(13, gt);
      ok = mbar_wait_warp(&bars[S_FULL + wg], own & 1u, abort_flag, lane);
      if (!ok) break;
      if (elected) GCA_TRACE(8, gt);
      tc_fence_after();
      uint32_t x[64];
      const uint32_t tS = tlane + (vs & 1u) * 128 + coff;       // accumulator g % 2
      tmem_ld_32x32b_x32(tS, x);
      tmem_ld_32x32b_x32(tS + 32, x + 32);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive_warp(&bars[K_FULL + kn], lane);    // the accumulator is free for slot g + 2
      if (elected) GCA_TRACE(9, gt);

      // row max: four independent chains of 3-input max
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
      if (GCA_DBG(1)) m0 = __uint_as_float(x[0]);
      else
#pragma unroll
      for (int cc = 0; cc < 64; cc += 8) {
        m0 = fmax3(m0, __uint_as_float(x[cc + 0]), __uint_as_float(x[cc + 1]));
        m1 = fmax3(m1, __uint_as_float(x[cc + 2]), __uint_as_float(x[cc + 3]));
        m2 = fmax3(m2, __uint_as_float(x[cc + 4]), __uint_as_float(x[cc + 5]));
        m3 = fmax3(m3, __uint_as_float(x[cc + 6]), __uint_as_float(x[cc + 7]));
      }
      float mm = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * p.c2;
      if (p.off_by_one > 0.f) mm = fmaxf(mm, 0.f);
      // p = exp2(x * c2 - mm): packed FMA, MUFU exp2, four packed partial sums
      const float2 c2v = make_float2(p.c2, p.c2), nmm = make_float2(-mm, -mm);
      float2 s0 = make_float2(0.f, 0.f), s1 = s0, s2 = s0, s3 = s0;
#pragma unroll
      for (int cc = 0; cc < 64; cc += 8) {
        float2 a0 = __ffma2_rn(make_float2(__uint_as_float(x[cc + 0]), __uint_as_float(x[cc + 1])), c2v, nmm);
        float2 a1 = __ffma2_rn(make_float2(__uint_as_float(x[cc + 2]), __uint_as_float(x[cc + 3])), c2v, nmm);
        float2 a2 = __ffma2_rn(make_float2(__uint_as_float(x[cc + 4]), __uint_as_float(x[cc + 5])), c2v, nmm);
        float2 a3 = __ffma2_rn(make_float2(__uint_as_float(x[cc + 6]), __uint_as_float(x[cc + 7])), c2v, nmm);
        if (!GCA_DBG(0)) {
        a0.x = ex2_approx(a0.x); a0.y = ex2_approx(a0.y);
        a1.x = ex2_approx(a1.x); a1.y = ex2_approx(a1.y);
        a2.x = ex2_approx(a2.x); a2.y = ex2_approx(a2.y);
        a3.x = ex2_approx(a3.x); a3.y = ex2_approx(a3.y);
        }
        s0 = __fadd2_rn(s0, a0); s1 = __fadd2_rn(s1, a1); s2 = __fadd2_rn(s2, a2); s3 = __fadd2_rn(s3, a3);
        x[cc + 0] = __float_as_uint(a0.x); x[cc + 1] = __float_as_uint(a0.y);
        x[cc + 2] = __float_as_uint(a1.x); x[cc + 3] = __float_as_uint(a1.y);
        x[cc + 4] = __float_as_uint(a2.x); x[cc + 5] = __float_as_uint(a2.y);
        x[cc + 6] = __float_as_uint(a3.x); x[cc + 7] = __float_as_uint(a3.y);
      }
      const float2 st2 = __fadd2_rn(__fadd2_rn(s0, s1), __fadd2_rn(s2, s3));
      float l = st2.x + st2.y;
      if (p.off_by_one > 0.f) l += p.off_by_one * ex2_approx(-mm);
      if (lse_base && live && !GCA_DBG(3)) lse_base[k * 64] = mm + __log2f(l);
      const float f = __fdividef(wk, l);
      const float2 fv = make_float2(f, f);

      if (elected) GCA_TRACE(10, gt);
      if (own > 0) {                                 // PV of this group's previous slot has consumed its P
        ok = mbar_wait_warp(&bars[P_EMPTY + wg], (own - 1) & 1u, abort_flag, lane);
        if (!ok) break;
      }
      if (elected) GCA_TRACE(11, gt);
      // P = (w / l) * exp2(...) in bf16, two per 32-bit column, straight into tensor memory: the
      // A operand of the PV product
      uint32_t pk[32];
#pragma unroll
      for (int cc = 0; cc < 32; cc += 4) {
        const float2 q0 = __fmul2_rn(make_float2(__uint_as_float(x[2 * cc + 0]), __uint_as_float(x[2 * cc + 1])), fv);
        const float2 q1 = __fmul2_rn(make_float2(__uint_as_float(x[2 * cc + 2]), __uint_as_float(x[2 * cc + 3])), fv);
        const float2 q2 = __fmul2_rn(make_float2(__uint_as_float(x[2 * cc + 4]), __uint_as_float(x[2 * cc + 5])), fv);
        const float2 q3 = __fmul2_rn(make_float2(__uint_as_float(x[2 * cc + 6]), __uint_as_float(x[2 * cc + 7])), fv);
        pk[cc + 0] = pack_bf16x2(q0.x, q0.y); pk[cc + 1] = pack_bf16x2(q1.x, q1.y);
        pk[cc + 2] = pack_bf16x2(q2.x, q2.y); pk[cc + 3] = pack_bf16x2(q3.x, q3.y);
      }
      if (!GCA_DBG(2)) {
        tmem_st_32x32b_x32(tP, pk);
        tmem_st_wait();
      }
      tc_fence_before();
      mbar_arrive_warp(&bars[V_FULL + vs], lane);    // "P of this slot is written"
      ++own;
      if (elected) GCA_TRACE(12, gt);
    }
    if (!ok) break;
    // epilogue by the group that had the unit's last slot: O tile -> bf16 -> global
    if (((flags >> DESC_EPI_SHIFT) & 3u) == (uint32_t)wg) {
#ifdef GCA_PROFILE
      const uint32_t g = g0 + __popc(umask);
#endif
      ok = mbar_wait_warp(&bars[O_FULL + wg], epi & 1, abort_flag, lane);
      ++epi;
      if (!ok) break;
      if (elected) GCA_TRACE(3, g - 1);
      tc_fence_after();
      // O leaves in four passes of ONE small loop body (16 columns: TMEM -> bf16 -> one 32-byte
      // store per row): after the first pass the body is in the instruction cache, where a
      // straight-line conversion of all 64 columns, executed once per unit, runs at
      // instruction-fetch speed (~10 cycles per instruction measured)
#pragma unroll 1
      for (int part = 0; part < 64 / OUT_COLS; ++part) {
        uint32_t v[OUT_COLS];
        if (OUT_COLS == 32) tmem_ld_32x32b_x32(tlane + TMEM_O + coff + part * OUT_COLS, v);
        else tmem_ld_32x32b_x16(tlane + TMEM_O + coff + part * OUT_COLS, v);
        tmem_ld_wait();
        if (live && !GCA_DBG(4)) {
#pragma unroll
          for (int h16 = 0; h16 < OUT_COLS / 16; ++h16) {
            uint32_t wv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i)
              wv[i] = pack_bf16x2(__uint_as_float(v[16 * h16 + 2 * i]), __uint_as_float(v[16 * h16 + 2 * i + 1]));
            uint8_t* dst = reinterpret_cast<uint8_t*>(orow) + part * OUT_COLS * 2 + h16 * 32;
            if (wide_store) st_global_256(dst, wv[0], wv[1], wv[2], wv[3], wv[4], wv[5], wv[6], wv[7]);
            else {
              reinterpret_cast<uint4*>(dst)[0] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
              reinterpret_cast<uint4*>(dst)[1] = make_uint4(wv[4], wv[5], wv[6], wv[7]);
            }
          }
        }
      }
      tc_fence_before();
      if (elected) GCA_TRACE(0, g - 1);
      mbar_arrive_warp(&bars[O_EMPTY], lane);
      if (elected) GCA_TRACE(6, g - 1);
    }
  }
}

__global__ void __launch_bounds__(NTHREADS, 1)
fwd_tc_kernel(const __grid_constant__ FwdTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + NUM_BARS + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[Q_FULL + i], 1); mbar_init(&bars[Q_EMPTY + i], 1); }
    for (int i = 0; i < NWG; ++i) { mbar_init(&bars[S_FULL + i], 1); mbar_init(&bars[P_EMPTY + i], 1); mbar_init(&bars[O_FULL + i], 1); }
    mbar_init(&bars[O_EMPTY], 4);
    for (int i = 0; i < ND; ++i) { mbar_init(&bars[DESC_FULL + i], 1); mbar_init(&bars[DESC_EMPTY + i], DESC_READERS); }
    for (int i = 0; i < NK; ++i) { mbar_init(&bars[K_FULL + i], 5); mbar_init(&bars[K_EMPTY + i], 1); }   // FULL: producer + 4 warps
    for (int i = 0; i < NV; ++i) { mbar_init(&bars[V_FULL + i], 5); mbar_init(&bars[V_EMPTY + i], 1); }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == SMMA_WARP) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  if (warp == KPROD_WARP && lane == 0) { tma_prefetch_desc(&p.tm_q); tma_prefetch_desc(&p.tm_k2); tma_prefetch_desc(&p.tm_k1); }
  if (warp == VPROD_WARP && lane == 0) { tma_prefetch_desc(&p.tm_v2); tma_prefetch_desc(&p.tm_v1); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < 4 * NWG) softmax_role(p, smem, bars, abort_flag, warp >> 2, warp & 3, lane, tmem_base);
  else if (warp == KPROD_WARP) kproducer_role(p, smem, bars, abort_flag, lane);
  else if (warp == VPROD_WARP) vproducer_role(p, smem, bars, abort_flag, lane);
  else if (warp == SMMA_WARP) issuer_role<0>(p, smem, bars, abort_flag, lane, tmem_base);
  else issuer_role<1>(p, smem, bars, abort_flag, lane, tmem_base);

  tc_fence_before();
  __syncthreads();
  if (warp == SMMA_WARP) tmem_dealloc(tmem_base, TMEM_COLS);
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
}

long long* g_profile_buffer = nullptr;

}  // namespace

void set_fwd_profile_buffer(void* device_ptr) { g_profile_buffer = static_cast<long long*>(device_ptr); }
long long* profile_buffer() { return g_profile_buffer; }

int launch_fwd_tc(const GcaFwdArgs& a, int sms, cudaStream_t stream) {
  if (a.dtype != GCA_BF16 || a.S != 64 || a.L != 64 || a.D != 64 || a.K > 32) return GCA_ERR_ALGO;
  FwdTcParams p;
  // q viewed as (d, s, h, j, n); caches as (d, l, h, c, n).  One copy moves a 64 x 64 tile of
  // each of two consecutive heads (box extent 2 on the head axis), or of one head (tm_*1).
  int rc;
  if ((rc = make_tile_map_5d(&p.tm_q, a.q, 64, 64, a.Hq, a.J, a.N, a.q_stride[3], a.q_stride[2], a.q_stride[1], a.q_stride[0], 2))) return rc;
  if ((rc = make_tile_map_5d(&p.tm_k2, a.k_cache, 64, 64, a.Hkv, a.C, a.N, a.k_stride[2], a.k_stride[3], a.k_stride[1], a.k_stride[0], 2))) return rc;
  if ((rc = make_tile_map_5d(&p.tm_v2, a.v_cache, 64, 64, a.Hkv, a.C, a.N, a.v_stride[2], a.v_stride[3], a.v_stride[1], a.v_stride[0], 2))) return rc;
  if ((rc = make_tile_map_5d(&p.tm_k1, a.k_cache, 64, 64, a.Hkv, a.C, a.N, a.k_stride[2], a.k_stride[3], a.k_stride[1], a.k_stride[0], 1))) return rc;
  if ((rc = make_tile_map_5d(&p.tm_v1, a.v_cache, 64, 64, a.Hkv, a.C, a.N, a.v_stride[2], a.v_stride[3], a.v_stride[1], a.v_stride[0], 1))) return rc;
  p.indices = a.indices; p.weights = a.weights; p.out = (__nv_bfloat16*)a.out; p.lse = a.lse; p.status = a.status;
  for (int i = 0; i < 4; ++i) p.os[i] = a.o_stride[i];
  p.N = a.N; p.J = a.J; p.Hq = a.Hq; p.Hkv = a.Hkv; p.G = a.Hq / a.Hkv; p.K = a.K; p.C = a.C;
  p.pair = a.algo == GCA_ALGO_TC_UNPAIRED ? 0 : 1;
  p.dbg = 0;
#ifdef GCA_DBGKNOBS
  if (const char* dbg_env = getenv("GCA_DBG")) p.dbg = atoi(dbg_env);      // timing experiments, never in the product build
#endif
  p.HP = p.pair ? (a.Hq + 1) / 2 : a.Hq;
  const long long units = (long long)a.N * a.J * p.HP;
  if (units >= (1ll << 31) - 65536) return GCA_ERR_TOO_LARGE;
  p.units = (int)units;
  p.c2 = a.sm_scale * GCA_LOG2E;
  p.off_by_one = a.off_by_one;
  p.prof = g_profile_buffer;
  p.wide_store = (reinterpret_cast<uintptr_t>(a.out) & 31u) == 0;
  for (int i = 0; i < 4; ++i) p.wide_store = p.wide_store && (a.o_stride[i] % 16 == 0);
  if (p.units == 0) return 0;
  GCA_CUDA_CHECK(cudaFuncSetAttribute(fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
  const unsigned grid = (unsigned)(p.units < sms ? p.units : sms);
  fwd_tc_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace gca
