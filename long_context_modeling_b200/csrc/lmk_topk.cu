// Landmark scoring + causal chunk mask + top-k + retrieval weights.
//
// The cached landmarks (E rows of D bf16 values) are streamed once.  One warp scores one
// landmark row at a time: the row is cut in 8-element (16-byte) pieces, lane l owns pieces
// l, l+32, l+64, ... so every load instruction of the warp covers 512 contiguous bytes.
// The float32 dot product is accumulated in a FIXED order (pieces in increasing order inside
// a lane, then a butterfly over the lanes), which makes every score -- and therefore every
// selected index -- independent of grid size, split count and GPU count.
//
// Candidates are 64-bit keys  orderable(score) << 32 | (0xFFFFFFFF - global_index):  a
// larger key is a better candidate, equal scores resolve to the lower index, and merging
// lists from warps, blocks or GPUs is a plain integer top-k.  Key 0 means "empty".
//
// Each warp keeps its running top-K per query row as a sorted list spread over its lanes
// (lane i holds the i-th best).  Blocks write their lists to a scratch buffer; a second,
// tiny kernel merges the lists of all blocks of a row and emits indices, noise-free scores,
// softmax weights and the number of valid slots.
#include "gca_common.cuh"

namespace gca {

namespace {

constexpr int SCAN_WARPS = 8;
constexpr int MAXK = 32;

__device__ __forceinline__ unsigned orderable(float s) {
  const unsigned u = __float_as_uint(s);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float from_orderable(unsigned o) {
  return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ unsigned long long make_key(float score, unsigned gidx) {
  return ((unsigned long long)orderable(score) << 32) | (unsigned long long)(0xffffffffu - gidx);
}
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// Insert `key` into the descending list held one element per lane.  Warp-uniform call.
__device__ __forceinline__ void list_insert(unsigned long long& mine, unsigned long long key, int lane) {
  const bool lower = mine < key;
  const unsigned long long up = __shfl_up_sync(0xffffffffu, mine, 1);
  const int lower_prev = __shfl_up_sync(0xffffffffu, (int)lower, 1);
  if (lower) mine = (lane > 0 && lower_prev) ? up : key;
}

__device__ __forceinline__ void unpack8(const uint4& v, float f[8]) {
  f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
  f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
  f[4] = __uint_as_float(v.z << 16); f[5] = __uint_as_float(v.z & 0xffff0000u);
  f[6] = __uint_as_float(v.w << 16); f[7] = __uint_as_float(v.w & 0xffff0000u);
}

struct ScanParams {
  const __nv_bfloat16* lq;
  const __nv_bfloat16* lk;
  const float* noise;
  unsigned long long* part;     // (rows, splits, K)
  long long qbs, qrs, kbs, krs;
  long long q_pos0, e_base;
  int N, Cq, E, D, K, H;
  int splits, e_per_split;
  int score_round;
  float scale;
};

// NP: pieces per lane (D <= 256*NP).  TQ: query rows per block (per-sequence mode).
// PER_HEAD: head_dim == 64, one list per head, TQ must be 1.
template <int NP, int TQ, bool PER_HEAD>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
lmk_scan_kernel(ScanParams p) {
  constexpr int NL = PER_HEAD ? NP * 4 : TQ;
  __shared__ unsigned long long sL[SCAN_WARPS][NL][MAXK];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, t0 = blockIdx.y * TQ, n = blockIdx.z;
  const int pieces = p.D >> 3;

  float qf[TQ][NP][8];
#pragma unroll
  for (int t = 0; t < TQ; ++t)
#pragma unroll
    for (int pp = 0; pp < NP; ++pp) {
      const int c = lane + 32 * pp;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (c < pieces && t0 + t < p.Cq)
        v = *reinterpret_cast<const uint4*>(p.lq + n * p.qbs + (long long)(t0 + t) * p.qrs + c * 8);
      unpack8(v, qf[t][pp]);
    }

  unsigned long long mine[NL];
  // Admission test: a candidate enters a full list only if its score beats the list's K-th
  // score (rows arrive in increasing index order inside a warp, so an equal score loses the
  // tie; scores are never -0).  NaN while the list is not full: "!(s <= NaN)" admits everything.
  float thr_s[PER_HEAD ? NP : TQ];
#pragma unroll
  for (int l = 0; l < NL; ++l) mine[l] = 0ull;
#pragma unroll
  for (int l = 0; l < (PER_HEAD ? NP : TQ); ++l) thr_s[l] = __int_as_float(0x7fc00000);

  const int e_lo = split * p.e_per_split;
  const int e_hi = min(p.E, e_lo + p.e_per_split);
  const __nv_bfloat16* kb = p.lk + n * p.kbs;
  // the last query row of the tile sees the most chunks: rows past that limit are skipped
  const long long tile_limit = p.q_pos0 + min(t0 + TQ, p.Cq) - 1;
  constexpr int U = (TQ == 1 && !PER_HEAD) ? 4 : 2;   // landmark rows in flight per warp iteration

  for (int e = e_lo + warp; e < e_hi; e += U * SCAN_WARPS) {
    uint4 kv[U][NP];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int eu = e + u * SCAN_WARPS;
#pragma unroll
      for (int pp = 0; pp < NP; ++pp) {
        const int c = lane + 32 * pp;
        kv[u][pp] = make_uint4(0, 0, 0, 0);
        if (eu < e_hi && c < pieces && p.e_base + eu < tile_limit)
          kv[u][pp] = *reinterpret_cast<const uint4*>(kb + (long long)eu * p.krs + c * 8);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int eu = e + u * SCAN_WARPS;
      const long long eg = p.e_base + eu;
      if (eu >= e_hi || eg >= tile_limit) continue;     // warp-uniform
      float kf[NP][8];
#pragma unroll
      for (int pp = 0; pp < NP; ++pp) unpack8(kv[u][pp], kf[pp]);
      if (!PER_HEAD) {
#pragma unroll
        for (int t = 0; t < TQ; ++t) {
          float acc = 0.f;
#pragma unroll
          for (int pp = 0; pp < NP; ++pp)
            if (lane + 32 * pp < pieces) {
#pragma unroll
              for (int jj = 0; jj < 8; ++jj) acc = fmaf(qf[t][pp][jj], kf[pp][jj], acc);
            }
#pragma unroll
          for (int of = 16; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
          float s = p.score_round ? round_bf16(round_bf16(acc) * p.scale) : acc * p.scale;
          const int row = t0 + t;
          const bool vis = row < p.Cq && eg < p.q_pos0 + row;
          if (p.noise && vis) s += p.noise[((long long)n * p.Cq + row) * p.E + eu];
          if (vis && !(s <= thr_s[t])) {
            list_insert(mine[t], make_key(s, (unsigned)eg), lane);
            const unsigned long long kth = __shfl_sync(0xffffffffu, mine[t], p.K - 1);
            if (kth != 0ull) thr_s[t] = from_orderable((unsigned)(kth >> 32));
          }
        }
      } else {
        const bool vis = eg < p.q_pos0 + t0;
#pragma unroll
        for (int pp = 0; pp < NP; ++pp) {
          float acc = 0.f;
          if (lane + 32 * pp < pieces) {
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) acc = fmaf(qf[0][pp][jj], kf[pp][jj], acc);
          }
#pragma unroll
          for (int of = 4; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
          // lanes 8g..8g+7 now hold the score of head 4*pp + g; each lane group tests it against
          // its own head's threshold, and only rows with a candidate take the uniform path
          const float s_loc = p.score_round ? round_bf16(round_bf16(acc) * p.scale) : acc * p.scale;
          const unsigned cand = __ballot_sync(0xffffffffu, vis && !(s_loc <= thr_s[pp]));
          if (cand == 0) continue;
#pragma unroll
          for (int hg = 0; hg < 4; ++hg) {
            if (!((cand >> (8 * hg)) & 1u)) continue;
            const int l = pp * 4 + hg;
            if (l >= p.H) continue;
            const float s = __shfl_sync(0xffffffffu, s_loc, hg * 8);
            list_insert(mine[l], make_key(s, (unsigned)eg), lane);
            const unsigned long long kth = __shfl_sync(0xffffffffu, mine[l], p.K - 1);
            if (kth != 0ull && (lane >> 3) == hg) thr_s[pp] = from_orderable((unsigned)(kth >> 32));
          }
        }
      }
    }
  }

  // merge the 8 per-warp lists of every row of the tile; list l is merged by warp l % 8
#pragma unroll
  for (int l = 0; l < NL; ++l)
    if (lane < p.K) sL[warp][l][lane] = mine[l];
  __syncthreads();
#pragma unroll
  for (int l = 0; l < NL; ++l) {
    if ((l % SCAN_WARPS) != warp) continue;
    long long row;
    if (PER_HEAD) { if (l >= p.H) continue; row = ((long long)n * p.Cq + t0) * p.H + l; }
    else          { if (t0 + l >= p.Cq) continue; row = (long long)n * p.Cq + t0 + l; }
    unsigned long long m = 0ull, th = 0ull;
    for (int w = 0; w < SCAN_WARPS; ++w)
      for (int i = 0; i < p.K; ++i) {
        const unsigned long long key = sL[w][l][i];
        if (key <= th) break;                              // lists are descending
        list_insert(m, key, lane);
        th = __shfl_sync(0xffffffffu, m, p.K - 1);
      }
    if (lane < p.K) p.part[(row * p.splits + split) * p.K + lane] = m;
  }
}

struct FinalParams {
  const unsigned long long* keys;   // (R, P)
  unsigned long long* out_keys;
  int32_t* out_indices;
  float* out_scores;
  float* out_weights;
  int32_t* out_nvalid;
  // optional recompute of noise-free scores (per-sequence mode with noise)
  const __nv_bfloat16* lq;
  const __nv_bfloat16* lk;
  long long qbs, qrs, kbs, krs, e_base;
  int Cq, D, score_round;
  float scale;
  int R, P, K;
};

constexpr int FIN_WARPS = 8;

// The merge of one row's P candidates (src) by one block of FIN_WARPS warps (sL: FIN_WARPS x MAXK
// keys of shared memory), and the decoded outputs of the row.
__device__ void finalize_row(const FinalParams& p, long long row, const unsigned long long* src,
                             unsigned long long (*sL)[MAXK]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // each warp merges a contiguous share of the candidates
  const int per = (p.P + FIN_WARPS - 1) / FIN_WARPS;
  const int lo = warp * per, hi = min(p.P, lo + per);
  unsigned long long m = 0ull, th = 0ull;
  for (int i0 = lo; i0 < hi; i0 += 32) {
    const unsigned long long mykey = (i0 + lane < hi) ? __ldcg(src + i0 + lane) : 0ull;   // may have been written by another GPU
    unsigned pending = __ballot_sync(0xffffffffu, mykey > th);
    while (pending) {
      const int srcl = __ffs(pending) - 1;
      pending &= pending - 1;
      const unsigned long long key = __shfl_sync(0xffffffffu, mykey, srcl);
      if (key > th) {
        list_insert(m, key, lane);
        th = __shfl_sync(0xffffffffu, m, p.K - 1);
      }
    }
  }
  if (lane < p.K) sL[warp][lane] = m;
  __syncthreads();
  if (warp != 0) return;
  m = 0ull; th = 0ull;
  for (int w = 0; w < FIN_WARPS; ++w)
    for (int i = 0; i < p.K; ++i) {
      const unsigned long long key = sL[w][i];
      if (key <= th) break;
      list_insert(m, key, lane);
      th = __shfl_sync(0xffffffffu, m, p.K - 1);
    }
  const bool valid = lane < p.K && m != 0ull;
  const int idx = valid ? (int)(0xffffffffu - (unsigned)(m & 0xffffffffull)) : -1;
  float score = valid ? from_orderable((unsigned)(m >> 32)) : -INFINITY;
  if (p.lq) {
    // selection used noisy scores: recompute the noise-free score of every winner in the
    // same fixed order as the scan
    const long long n = row / p.Cq, r = row % p.Cq;
    const int pieces = p.D >> 3;
    for (int i = 0; i < p.K; ++i) {
      const int wi = __shfl_sync(0xffffffffu, idx, i);
      if (wi < 0) continue;
      float acc = 0.f;
      for (int c = lane; c < pieces; c += 32) {
        const uint4 a = *reinterpret_cast<const uint4*>(p.lq + n * p.qbs + r * p.qrs + c * 8);
        const uint4 b = *reinterpret_cast<const uint4*>(p.lk + n * p.kbs + (wi - p.e_base) * p.krs + c * 8);
        float af[8], bf[8];
        unpack8(a, af); unpack8(b, bf);
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) acc = fmaf(af[jj], bf[jj], acc);
      }
#pragma unroll
      for (int of = 16; of > 0; of >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, of);
      const float s = p.score_round ? round_bf16(round_bf16(acc) * p.scale) : acc * p.scale;
      if (lane == i) score = s;
    }
  }
  // softmax over the valid slots
  float mx = valid ? score : -INFINITY;
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
  float ex = valid ? expf(score - mx) : 0.f;
  float sum = ex;
#pragma unroll
  for (int of = 16; of > 0; of >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, of);
  const float wgt = (valid && sum > 0.f) ? ex / sum : 0.f;
  const unsigned nv = __popc(__ballot_sync(0xffffffffu, valid));
  if (lane < p.K) {
    const long long o = row * p.K + lane;
    if (p.out_keys) p.out_keys[o] = m;
    if (p.out_indices) p.out_indices[o] = idx;
    if (p.out_scores) p.out_scores[o] = score;
    if (p.out_weights) p.out_weights[o] = wgt;
  }
  if (lane == 0 && p.out_nvalid) p.out_nvalid[row] = (int)nv;
}

__global__ void __launch_bounds__(FIN_WARPS * 32)
lmk_finalize_kernel(FinalParams p) {
  __shared__ unsigned long long sL[FIN_WARPS][MAXK];
  finalize_row(p, blockIdx.x, p.keys + (long long)blockIdx.x * p.P, sL);
}

// ---------------------------------------------------------------------------------------------
// Candidate exchange between the GPUs of a chunk-range-sharded cache, fused with the merge.
//
// Every rank owns a MAILBOX in its own memory that the other ranks of the node have mapped
// (CUDA IPC).  One launch per rank and retrieval step: a block per query row
//   1. STORES this rank's K packed candidates of the row into its slot of every rank's mailbox
//      (plain stores through the peer mapping; over NVLink for the other GPUs),
//   2. raises its flag there (system-scope release after a system-scope fence),
//   3. waits -- for at most `wait_ns` -- until every rank's flag of this step stands in its OWN
//      mailbox (system-scope acquire loads of local memory),
//   4. merges the world x K candidates (same merge, same canonical order as on one GPU, so every
//      rank gets the identical result) and writes indices / scores / weights.
// No rank reads another GPU's memory and nothing is multicast: remote traffic is stores only.
// Steps are numbered by an epoch the kernel keeps in the mailbox header (one per row, advanced
// when the row's merge is done), so the launch can sit in a CUDA graph; two mailbox buffers
// alternate by epoch parity: a rank can be at most one step ahead of another (to finish step e
// it needs everybody's flag of step e), so a buffer is never overwritten while it is being read.
// When the wait expires the block raises GCA_STATUS_TIMEOUT, leaves the epoch where it was and
// returns: the context stays usable, and the host decides (PeerExchange.reset()).
//
// Mailbox layout (bytes): epoch[R_max] u32 | pad to 256 | 2 x { keys[R_max][world][MAXK] u64 |
// flags[R_max][world] u32 | pad to 256 }.
struct ExchangeParams {
  const unsigned long long* local_keys;     // (R, K)
  void* const* mailboxes;                   // device array of `world` pointers (this process's mappings)
  FinalParams fin;
  int32_t* status;
  int R, K, world, rank, r_max;
  unsigned long long wait_ns;
};

__host__ __device__ inline size_t exch_buf_bytes(int r_max, int world) {
  const size_t keys = (size_t)r_max * world * MAXK * 8, flags = (size_t)r_max * world * 4;
  return (keys + flags + 255) / 256 * 256;
}
__host__ __device__ inline size_t exch_hdr_bytes(int r_max) { return ((size_t)r_max * 4 + 255) / 256 * 256; }

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__global__ void __launch_bounds__(FIN_WARPS * 32)
lmk_exchange_kernel(ExchangeParams p) {
  __shared__ unsigned long long sL[FIN_WARPS][MAXK];
  __shared__ int s_ok;
  const int row = blockIdx.x, tid = threadIdx.x;
  char* mine = static_cast<char*>(p.mailboxes[p.rank]);
  unsigned* epochs = reinterpret_cast<unsigned*>(mine);
  const unsigned e = *reinterpret_cast<volatile unsigned*>(epochs + row) + 1u;
  const size_t buf_off = exch_hdr_bytes(p.r_max) + (size_t)(e & 1u) * exch_buf_bytes(p.r_max, p.world);
  const size_t flags_off = buf_off + (size_t)p.r_max * p.world * MAXK * 8;
  // 1. my candidates into my slot of every rank's mailbox (thread = (destination rank, key); a
  //    slot is MAXK keys wide, the keys past K are written as "empty")
  if (tid < p.world * MAXK) {
    const int dst = tid / MAXK, i = tid - dst * MAXK;
    unsigned long long* slot = reinterpret_cast<unsigned long long*>(static_cast<char*>(p.mailboxes[dst]) + buf_off) +
                               ((size_t)row * p.world + p.rank) * MAXK;
    slot[i] = i < p.K ? p.local_keys[(size_t)row * p.K + i] : 0ull;
  }
  __threadfence_system();
  __syncthreads();
  // 2. my flag of this step in every rank's mailbox
  if (tid < p.world) {
    unsigned* flag = reinterpret_cast<unsigned*>(static_cast<char*>(p.mailboxes[tid]) + flags_off) + (size_t)row * p.world + p.rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(e) : "memory");
  }
  // 3. bounded wait for every rank's flag in MY mailbox
  if (tid == 0) s_ok = 1;
  __syncthreads();
  if (tid < p.world) {
    const unsigned* flag = reinterpret_cast<const unsigned*>(mine + flags_off) + (size_t)row * p.world + tid;
    const unsigned long long t0 = global_ns();
    for (;;) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
      if (v == e) break;
      if (global_ns() - t0 > p.wait_ns) { s_ok = 0; break; }
      __nanosleep(200);
    }
  }
  __syncthreads();
  if (!s_ok) {
    if (tid == 0 && p.status) atomicOr(p.status, GCA_STATUS_TIMEOUT);
    return;
  }
  // 4. the row's candidates sit contiguously in my mailbox, MAXK per rank with empty keys (0) as
  //    filler: the merge takes them in place as P = world x MAXK candidates
  const unsigned long long* src = reinterpret_cast<const unsigned long long*>(mine + buf_off) + (size_t)row * p.world * MAXK;
  finalize_row(p.fin, row, src, sL);
  if (tid == 0) epochs[row] = e;
}

// Two CTAs per SM when the query tile count alone does not fill the GPU.
int choose_splits(const LmkTopkArgs& a, int tq, int sms) {
  if (a.splits > 0) return a.splits;
  const long long blocks = (long long)a.N * ((a.Cq + tq - 1) / tq);
  long long s = (2 * (long long)sms + blocks - 1) / blocks;
  const long long max_s = (a.E + 255) / 256;              // keep at least 256 rows per split
  if (s > max_s) s = max_s;
  if (s < 1) s = 1;
  return (int)s;
}

int pick_tq(const LmkTopkArgs& a) { return (a.head_dim > 0 || a.Cq < 4) ? 1 : 4; }

template <int NP>
void launch_scan(const ScanParams& sp, int tq, bool per_head, dim3 grid, cudaStream_t stream) {
  if (per_head) lmk_scan_kernel<NP, 1, true><<<grid, SCAN_WARPS * 32, 0, stream>>>(sp);
  else if (tq == 1) lmk_scan_kernel<NP, 1, false><<<grid, SCAN_WARPS * 32, 0, stream>>>(sp);
  else lmk_scan_kernel<NP, 4, false><<<grid, SCAN_WARPS * 32, 0, stream>>>(sp);
}

}  // namespace

size_t lmk_topk_rows(const LmkTopkArgs& a) {
  const int H = a.head_dim > 0 ? a.D / a.head_dim : 1;
  return (size_t)a.N * a.Cq * H;
}

size_t lmk_topk_workspace_bytes_impl(const LmkTopkArgs& a, int sms) {
  const int splits = choose_splits(a, pick_tq(a), sms);
  return align_up(lmk_topk_rows(a) * (size_t)splits * a.K * sizeof(unsigned long long), 256);
}

// Scan + finalize on caller-provided scratch.  `scratch` must hold
// lmk_topk_workspace_bytes_impl(a, sms) bytes.
int launch_lmk_score_topk(const LmkTopkArgs& a, void* scratch, int sms, cudaStream_t stream) {
  const bool per_head = a.head_dim > 0;
  const int H = per_head ? a.D / a.head_dim : 1;
  const int tq = pick_tq(a);
  const int splits = choose_splits(a, tq, sms);
  ScanParams sp;
  sp.lq = (const __nv_bfloat16*)a.lmk_q; sp.lk = (const __nv_bfloat16*)a.lmk_k; sp.noise = a.noise;
  sp.part = (unsigned long long*)scratch;
  sp.qbs = a.q_batch_stride; sp.qrs = a.q_row_stride; sp.kbs = a.k_batch_stride; sp.krs = a.k_row_stride;
  sp.q_pos0 = a.q_pos0; sp.e_base = a.e_base;
  sp.N = a.N; sp.Cq = a.Cq; sp.E = a.E; sp.D = a.D; sp.K = a.K; sp.H = H;
  sp.splits = splits; sp.e_per_split = (a.E + splits - 1) / splits;
  sp.score_round = a.score_round;
  sp.scale = (float)(1.0 / sqrt((double)(per_head ? a.head_dim : a.D)));
  const size_t rows = lmk_topk_rows(a);
  if (rows == 0) return 0;
  dim3 grid((unsigned)splits, (unsigned)((a.Cq + tq - 1) / tq), (unsigned)a.N);
  const int np = (a.D + 255) / 256;
  switch (np) {
    case 1: launch_scan<1>(sp, tq, per_head, grid, stream); break;
    case 2: launch_scan<2>(sp, tq, per_head, grid, stream); break;
    case 3: launch_scan<3>(sp, tq, per_head, grid, stream); break;
    case 4: launch_scan<4>(sp, tq, per_head, grid, stream); break;
    default: return GCA_ERR_SHAPE;
  }
  GCA_CUDA_CHECK(cudaGetLastError());
  FinalParams fp;
  fp.keys = sp.part; fp.out_keys = (unsigned long long*)a.out_keys; fp.out_indices = a.out_indices; fp.out_scores = a.out_scores;
  fp.out_weights = a.out_weights; fp.out_nvalid = a.out_nvalid;
  const bool recompute = a.noise != nullptr && !per_head;
  fp.lq = recompute ? sp.lq : nullptr; fp.lk = sp.lk;
  fp.qbs = sp.qbs; fp.qrs = sp.qrs; fp.kbs = sp.kbs; fp.krs = sp.krs; fp.e_base = a.e_base;
  fp.Cq = a.Cq; fp.D = a.D; fp.score_round = a.score_round; fp.scale = sp.scale;
  fp.R = (int)rows; fp.P = splits * a.K; fp.K = a.K;
  lmk_finalize_kernel<<<(unsigned)rows, FIN_WARPS * 32, 0, stream>>>(fp);
  return (int)cudaGetLastError();
}

int launch_lmk_merge(const LmkMergeArgs& a, cudaStream_t stream) {
  if (a.R == 0) return 0;
  FinalParams fp;
  fp.keys = (const unsigned long long*)a.keys; fp.out_keys = (unsigned long long*)a.out_keys; fp.out_indices = a.out_indices; fp.out_scores = a.out_scores;
  fp.out_weights = a.out_weights; fp.out_nvalid = a.out_nvalid;
  fp.lq = nullptr; fp.lk = nullptr; fp.qbs = fp.qrs = fp.kbs = fp.krs = fp.e_base = 0;
  fp.Cq = 1; fp.D = 0; fp.score_round = 0; fp.scale = 1.f;
  fp.R = a.R; fp.P = a.P; fp.K = a.K;
  lmk_finalize_kernel<<<(unsigned)a.R, FIN_WARPS * 32, 0, stream>>>(fp);
  return (int)cudaGetLastError();
}

}  // namespace gca

// ---------------------------------------------------------------------------------------------
// lmk_score_topk_static: the same scan + finalize, for callers that cannot hand us scratch.
//
// Who needs this: a host that must not (or cannot) allocate device memory around the call --
// for example a serving process that gave all of HBM to its own pools at start-up, a plugin
// living inside another framework whose allocator it may not touch, or a latency-critical loop
// where an allocator call (and the device-wide synchronisation it can imply) is not acceptable.
// Such a caller still passes its inputs and outputs, but the per-block candidate lists go into
// a fixed array that lives in the library image.
//
// The array is file-scope device memory: every GPU that loads this library carries it
// (LMK_STATIC_SCRATCH_BYTES = 1 MiB) until the process exits.  In host code its name is only a
// stand-in for the symbol, not a device address, so the address is looked up with
// cudaGetSymbolAddress -- once per device, with that device current (the device that holds the
// landmark cache, made current for the call), on the first call made for that device -- and only
// that looked-up pointer is handed to the kernels.  Because of that
// look-up, make the first call on each device before starting any stream capture.
//
// All calls on one GPU share the array.  It keeps whatever the previous call left in it; that
// is harmless here because a call writes every (row, split) list it later reads, so nothing
// needs to start at zero.  Two calls that overlap on the same GPU (different streams, or
// different host threads) would overwrite each other's lists: serialise them.
// ---------------------------------------------------------------------------------------------
#include <cstring>
#include <mutex>

namespace gca {
namespace {

static __device__ __align__(256) unsigned long long g_lmk_static_scratch[LMK_STATIC_SCRATCH_BYTES / 8];

constexpr int MAX_DEVICES = 64;
std::mutex g_static_mu;
void* g_static_ptr[MAX_DEVICES] = {};

// Device address of the static scratch on device `dev`, which must be current (resolved once per device).
int static_scratch_ptr(int dev, void** out) {
  if (dev < 0 || dev >= MAX_DEVICES) return GCA_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ptr[dev]) {
    void* p = nullptr;
    GCA_CUDA_CHECK(cudaGetSymbolAddress(&p, g_lmk_static_scratch));
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return 0;
}

}  // namespace
}  // namespace gca

extern "C" int lmk_score_topk_static(const LmkTopkArgs* a, void* stream) {
  // same argument rules as lmk_score_topk; `workspace` / `workspace_bytes` are ignored
  int rc = gca::check_topk(a);
  if (rc) return rc;
  if (a->N == 0 || a->Cq == 0) return 0;
  gca::DeviceScope scope(a->lmk_k);        // the array of the GPU that holds the landmarks
  if (scope.rc) return scope.rc;
  const int sms = gca::sm_count(scope.dev);
  // rows x splits x K candidate keys of 8 bytes must fit the built-in array
  if (gca::lmk_topk_workspace_bytes_impl(*a, sms) > (size_t)LMK_STATIC_SCRATCH_BYTES) return GCA_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  rc = gca::static_scratch_ptr(scope.dev, &scratch);
  if (rc) return rc;
  return gca::launch_lmk_score_topk(*a, scratch, sms, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------
// Host side of the candidate exchange: mailbox set-up (CUDA IPC) and the launch.
// ---------------------------------------------------------------------------------------------
extern "C" size_t lmk_exchange_mailbox_bytes(int r_max, int world) {
  if (r_max < 1 || world < 1) return 0;
  return gca::exch_hdr_bytes(r_max) + 2 * gca::exch_buf_bytes(r_max, world);
}

extern "C" int lmk_exchange_mailbox_create(int r_max, int world, void** mailbox, void* ipc_handle64) {
  if (!mailbox || !ipc_handle64) return GCA_ERR_NULL;
  if (r_max < 1 || world < 1 || world > 8) return GCA_ERR_SHAPE;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  const size_t bytes = lmk_exchange_mailbox_bytes(r_max, world);
  void* p = nullptr;
  GCA_CUDA_CHECK(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle64), p);
  if (e != cudaSuccess) { cudaFree(p); return (int)e; }
  *mailbox = p;
  return 0;
}

extern "C" int lmk_exchange_mailbox_open(const void* ipc_handle64, void** peer_ptr) {
  if (!ipc_handle64 || !peer_ptr) return GCA_ERR_NULL;
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle64, sizeof(h));
  GCA_CUDA_CHECK(cudaIpcOpenMemHandle(peer_ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}

extern "C" int lmk_exchange_mailbox_close(void* peer_ptr) {
  if (!peer_ptr) return GCA_ERR_NULL;
  GCA_CUDA_CHECK(cudaIpcCloseMemHandle(peer_ptr));
  return 0;
}

extern "C" int lmk_exchange_mailbox_destroy(void* mailbox) {
  if (!mailbox) return GCA_ERR_NULL;
  GCA_CUDA_CHECK(cudaFree(mailbox));
  return 0;
}

extern "C" int lmk_exchange_mailbox_reset(void* mailbox, int r_max, int world, void* stream) {
  if (!mailbox) return GCA_ERR_NULL;
  GCA_CUDA_CHECK(cudaMemsetAsync(mailbox, 0, lmk_exchange_mailbox_bytes(r_max, world), (cudaStream_t)stream));
  return 0;
}

extern "C" int lmk_topk_exchange(const LmkExchangeArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->local_keys || !a->mailboxes || !a->out_keys) return GCA_ERR_NULL;
  if (a->world < 1 || a->world > 8 || a->rank < 0 || a->rank >= a->world) return GCA_ERR_SHAPE;
  if (a->R < 0 || a->R > a->R_max || a->K < 1 || a->K > gca::MAXK) return GCA_ERR_SHAPE;
  if (a->R == 0) return 0;
  gca::DeviceScope scope(a->local_keys);
  if (scope.rc) return scope.rc;
  gca::ExchangeParams p;
  p.local_keys = reinterpret_cast<const unsigned long long*>(a->local_keys);
  p.mailboxes = a->mailboxes;
  p.status = a->status;
  p.R = a->R; p.K = a->K; p.world = a->world; p.rank = a->rank; p.r_max = a->R_max;
  p.wait_ns = (unsigned long long)(a->wait_ms > 0 ? a->wait_ms : 1000) * 1000000ull;
  gca::FinalParams& fp = p.fin;
  fp.keys = nullptr; fp.out_keys = reinterpret_cast<unsigned long long*>(a->out_keys); fp.out_indices = a->out_indices;
  fp.out_scores = a->out_scores; fp.out_weights = a->out_weights; fp.out_nvalid = a->out_nvalid;
  fp.lq = nullptr; fp.lk = nullptr; fp.qbs = fp.qrs = fp.kbs = fp.krs = fp.e_base = 0;
  fp.Cq = 1; fp.D = 0; fp.score_round = 0; fp.scale = 1.f;
  fp.R = a->R; fp.P = a->world * gca::MAXK; fp.K = a->K;
  gca::lmk_exchange_kernel<<<(unsigned)a->R, gca::FIN_WARPS * 32, 0, (cudaStream_t)stream>>>(p);
  return (int)cudaGetLastError();
}
