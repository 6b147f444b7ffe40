// extern "C" entry points of libgca_b200.so: argument validation on the host, kernel
// selection, launches on the caller's stream.  Nothing here allocates device memory.
#include <mutex>

#include "gca_common.cuh"

namespace gca {
int launch_decode(const GcaFwdArgs& a, int sms, cudaStream_t stream);
int launch_lmk_score_topk(const LmkTopkArgs& a, void* scratch, int sms, cudaStream_t stream);
int launch_lmk_merge(const LmkMergeArgs& a, cudaStream_t stream);
size_t lmk_topk_workspace_bytes_impl(const LmkTopkArgs& a, int sms);
bool bwd_tc_available();
void set_fwd_profile_buffer(void* device_ptr);
int launch_cache_append(const CacheAppendArgs& a, cudaStream_t stream);
int launch_kv_project_append(const KvProjectArgs& a, int sms, cudaStream_t stream);
int launch_row_rms(const RowRmsArgs& a, cudaStream_t stream);
int launch_silu_mul(const void* gu, void* out, long long M, int I, long long in_stride, long long out_stride, cudaStream_t stream);
int launch_linear(const LinearArgs& a, int sms, cudaStream_t stream);
int launch_window_decode(const WindowDecodeArgs& a, cudaStream_t stream);
int launch_window_ring_decode(const WindowRingDecodeArgs& a, cudaStream_t stream);
int launch_linear_ce(const LinearCeArgs& a, int sms, cudaStream_t stream);
int launch_window_shift_append(const WindowAppendArgs& a, cudaStream_t stream);

DeviceScope::DeviceScope(const void* device_ptr) {
  cudaPointerAttributes at;
  cudaError_t e = cudaPointerGetAttributes(&at, device_ptr);
  if (e != cudaSuccess) { rc = (int)e; (void)cudaGetLastError(); return; }
  if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged) { rc = GCA_ERR_NULL; return; }   // not device memory
  dev = at.device;
  if ((e = cudaGetDevice(&prev)) != cudaSuccess) { rc = (int)e; prev = -1; return; }
  if (prev != dev && (e = cudaSetDevice(dev)) != cudaSuccess) { rc = (int)e; prev = -1; }
}
DeviceScope::~DeviceScope() {
  if (prev >= 0 && prev != dev) (void)cudaSetDevice(prev);
}

int sm_count(int dev) {
  constexpr int MAXD = 64;
  static std::mutex mu;
  static int cached[MAXD] = {};
  if (dev < 0 || dev >= MAXD) return 1;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
    cached[dev] = n;
  }
  return cached[dev];
}
}  // namespace gca

namespace {

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int esize_of(int dtype) { return dtype == GCA_BF16 ? 2 : dtype == GCA_F32 ? 4 : 0; }

// Strides of the four outer axes must keep every row 16-byte aligned.
int check_strides(const int64_t s[4], int esize, const int32_t dims[4]) {
  for (int i = 0; i < 4; ++i) {
    if (dims[i] > 1 || i == 3) {
      if (s[i] < 0) return GCA_ERR_STRIDE;
      if (((long long)s[i] * esize) % 16 != 0) return GCA_ERR_STRIDE;
    }
  }
  return 0;
}

int check_common(const void* q, const void* k, const void* v, const int32_t* idx, const float* w, int dtype, int N,
                 int J, int Hq, int Hkv, int S, int L, int D, int K, int C) {
  if (!q || !k || !v || !idx || !w) return GCA_ERR_NULL;
  if (esize_of(dtype) == 0) return GCA_ERR_DTYPE;
  if (N < 0 || J < 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return GCA_ERR_SHAPE;
  if (L != 64 || D != 64 || S < 1 || S > 64 || K < 1 || K > 32 || C < 1) return GCA_ERR_SHAPE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v)) return GCA_ERR_ALIGN;
  return 0;
}

int check_fwd(const GcaFwdArgs* a) {
  if (!a) return GCA_ERR_NULL;
  int rc = check_common(a->q, a->k_cache, a->v_cache, a->indices, a->weights, a->dtype, a->N, a->J, a->Hq, a->Hkv,
                        a->S, a->L, a->D, a->K, a->C);
  if (rc) return rc;
  if (!a->out) return GCA_ERR_NULL;
  if (!aligned16(a->out)) return GCA_ERR_ALIGN;
  if (!(a->sm_scale > 0.f) || a->off_by_one < 0.f) return GCA_ERR_SHAPE;
  const int es = esize_of(a->dtype);
  const int32_t qd[4] = {a->N, a->J, a->Hq, a->S};
  const int32_t kd[4] = {a->N, a->C, a->L, a->Hkv};
  if ((rc = check_strides(a->q_stride, es, qd))) return rc;
  if ((rc = check_strides(a->o_stride, es, qd))) return rc;
  if ((rc = check_strides(a->k_stride, es, kd))) return rc;
  if ((rc = check_strides(a->v_stride, es, kd))) return rc;
  return 0;
}

}  // namespace

extern "C" {

int gca_abi_version(void) { return GCA_ABI_VERSION; }

#ifdef GCA_PROFILE
// Profile builds only (never declared in the public header): a device buffer of 64 + 16 * 256
// int64 words into which block 0 of the tensor-core kernels records event clocks; NULL = off.
int gca_debug_profile_buffer(void* device_ptr) {
  gca::set_fwd_profile_buffer(device_ptr);
  return 0;
}
#endif

size_t gca_sizeof(int which) {
  switch (which) {
    case 0: return sizeof(GcaFwdArgs);
    case 1: return sizeof(GcaBwdArgs);
    case 2: return sizeof(LmkTopkArgs);
    case 3: return sizeof(LmkMergeArgs);
    case 4: return sizeof(CacheAppendArgs);
    case 5: return sizeof(LmkExchangeArgs);
    case 6: return sizeof(KvProjectArgs);
    case 7: return sizeof(RowRmsArgs);
    case 8: return sizeof(LinearArgs);
    case 9: return sizeof(WindowDecodeArgs);
    case 10: return sizeof(LinearCeArgs);
    case 11: return sizeof(WindowAppendArgs);
    case 12: return sizeof(WindowRingDecodeArgs);
    default: return 0;
  }
}

const char* gca_strerror(int code) {
  switch (code) {
    case GCA_OK: return "ok";
    case GCA_ERR_NULL: return "a required pointer is NULL";
    case GCA_ERR_DTYPE: return "unsupported dtype";
    case GCA_ERR_SHAPE: return "dimension outside the supported envelope (L = D = 64, 1 <= S <= 64, 1 <= K <= 32, Hq % Hkv == 0)";
    case GCA_ERR_STRIDE: return "stride not usable: rows must stay 16-byte aligned";
    case GCA_ERR_ALIGN: return "base pointer not 16-byte aligned";
    case GCA_ERR_WORKSPACE: return "workspace missing or too small";
    case GCA_ERR_ALGO: return "requested kernel variant cannot run this problem";
    case GCA_ERR_TMA: return "tensor-map encoding rejected by the driver";
    case GCA_ERR_TOO_LARGE: return "size exceeds a fixed built-in limit";
    case GCA_ERR_STATIC_SCRATCH:
      return "lmk_score_topk_static: rows * splits * K * 8 bytes exceeds the 1 MiB built-in scratch "
             "(lower args->splits or use lmk_score_topk with a workspace)";
    default: break;
  }
  if (code > 0) return cudaGetErrorString((cudaError_t)code);
  return "unknown error";
}

int gca_fwd(const GcaFwdArgs* a, void* stream) {
  int rc = check_fwd(a);
  if (rc) return rc;
  if (a->N == 0 || a->J == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  gca::DeviceScope scope(a->q);
  if (scope.rc) return scope.rc;
  int algo = a->algo;
  const bool tc_ok = a->dtype == GCA_BF16 && a->S == 64;
  if (algo == GCA_ALGO_AUTO) algo = tc_ok ? GCA_ALGO_TC : GCA_ALGO_SIMT;
  if (algo == GCA_ALGO_TC || algo == GCA_ALGO_TC_UNPAIRED) {
    if (!tc_ok) return GCA_ERR_ALGO;
    GcaFwdArgs b = *a;
    b.algo = algo;
    return gca::launch_fwd_tc(b, gca::sm_count(scope.dev), s);
  }
  if (algo == GCA_ALGO_SIMT) return gca::launch_fwd_simt(*a, s);
  return GCA_ERR_ALGO;
}

int gca_decode(const GcaFwdArgs* a, void* stream) {
  int rc = check_fwd(a);
  if (rc) return rc;
  if (a->S > 16) return GCA_ERR_SHAPE;
  if (a->N == 0 || a->J == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  gca::DeviceScope scope(a->q);
  if (scope.rc) return scope.rc;
  if (a->algo != GCA_ALGO_SIMT && a->dtype == GCA_BF16 && (a->Hq / a->Hkv) * a->S <= 16)
    return gca::launch_decode(*a, gca::sm_count(scope.dev), s);
  if (a->algo == GCA_ALGO_TC || a->algo == GCA_ALGO_TC_UNPAIRED) return GCA_ERR_ALGO;
  GcaFwdArgs b = *a;
  b.lse = nullptr;
  return gca::launch_fwd_simt(b, s);
}

static size_t dw_part_bytes(const GcaBwdArgs* a) {
  return gca::align_up((size_t)4 * a->N * a->J * a->Hq * a->K * sizeof(float), 256);   // up to four partials per (row block, head, slot)
}

// 16 bytes per (row block, head, slot, row): written by the q-major pass, read by the kv-major pass
static size_t rowterm_bytes(const GcaBwdArgs* a) {
  return gca::align_up((size_t)a->N * a->J * a->Hq * a->K * 64 * sizeof(uint4), 256);
}

size_t gca_bwd_workspace_bytes(const GcaBwdArgs* a) {
  if (!a) return 0;
  return gca::csr_workspace_bytes(a->N, a->J, a->K, a->C) + dw_part_bytes(a) + rowterm_bytes(a);
}

int gca_bwd(const GcaBwdArgs* a, void* stream) { return gca_bwd_stages(a, GCA_BWD_STAGE_ALL, stream); }

int gca_bwd_stages(const GcaBwdArgs* a, unsigned stages, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if ((stages & (unsigned)GCA_BWD_STAGE_ALL) == 0 || (stages & ~(unsigned)(GCA_BWD_STAGE_ALL | GCA_BWD_INDEX_BY_SORT)))
    return GCA_ERR_SHAPE;
  int rc = check_common(a->q, a->k_cache, a->v_cache, a->indices, a->weights, a->dtype, a->N, a->J, a->Hq, a->Hkv,
                        a->S, a->L, a->D, a->K, a->C);
  if (rc) return rc;
  if (!a->dout || !a->lse || !a->dq || !a->dk_cache || !a->dv_cache || !a->dw) return GCA_ERR_NULL;
  if (!aligned16(a->dout) || !aligned16(a->dq) || !aligned16(a->dk_cache) || !aligned16(a->dv_cache)) return GCA_ERR_ALIGN;
  if (!(a->sm_scale > 0.f) || a->off_by_one < 0.f) return GCA_ERR_SHAPE;
  const int es = esize_of(a->dtype);
  const int32_t qd[4] = {a->N, a->J, a->Hq, a->S};
  const int32_t kd[4] = {a->N, a->C, a->L, a->Hkv};
  if ((rc = check_strides(a->q_stride, es, qd))) return rc;
  if ((rc = check_strides(a->do_stride, es, qd))) return rc;
  if ((rc = check_strides(a->dq_stride, es, qd))) return rc;
  if ((rc = check_strides(a->k_stride, es, kd))) return rc;
  if ((rc = check_strides(a->v_stride, es, kd))) return rc;
  if ((rc = check_strides(a->dk_stride, es, kd))) return rc;
  if ((rc = check_strides(a->dv_stride, es, kd))) return rc;
  if (a->N == 0) return 0;
  if (!a->workspace || (reinterpret_cast<uintptr_t>(a->workspace) & 255u)) return GCA_ERR_WORKSPACE;
  if (a->workspace_bytes < gca_bwd_workspace_bytes(a)) return GCA_ERR_WORKSPACE;
  cudaStream_t s = (cudaStream_t)stream;
  gca::DeviceScope scope(a->q);
  if (scope.rc) return scope.rc;
  gca::Csr csr;
  size_t used = 0;
  rc = gca::build_csr(a->indices, a->N, a->J, a->K, a->C, a->workspace, a->workspace_bytes, &csr, &used, s,
                      (stages & GCA_BWD_STAGE_INDEX) != 0, (stages & GCA_BWD_INDEX_BY_SORT) != 0);
  if (rc) return rc;
  if (!(stages & (GCA_BWD_STAGE_KV | GCA_BWD_STAGE_Q))) return 0;
  float* dw_part = reinterpret_cast<float*>(static_cast<char*>(a->workspace) + used);
  uint4* rowterm = reinterpret_cast<uint4*>(static_cast<char*>(a->workspace) + used + dw_part_bytes(a));
  int algo = a->algo;
  const bool tc_ok = a->dtype == GCA_BF16 && a->S == 64;
  if (algo == GCA_ALGO_TC_UNPAIRED) algo = GCA_ALGO_TC;
  if (algo == GCA_ALGO_AUTO) algo = tc_ok ? GCA_ALGO_TC : GCA_ALGO_SIMT;
  if (algo == GCA_ALGO_TC)
    rc = tc_ok ? gca::launch_bwd_tc(*a, csr, dw_part, rowterm, gca::sm_count(scope.dev), s, stages & GCA_BWD_STAGE_ALL) : GCA_ERR_ALGO;
  else if (algo == GCA_ALGO_SIMT) rc = gca::launch_bwd_simt(*a, csr, dw_part, s, stages & GCA_BWD_STAGE_ALL);
  else rc = GCA_ERR_ALGO;
  if (rc) return rc;
  if (!(stages & GCA_BWD_STAGE_Q)) return 0;
  return gca::launch_dw_reduce(dw_part, a->dw, a->N * a->J, a->Hq, a->K, algo == GCA_ALGO_TC ? gca::bwd_tc_dw_parts() : 1, s);
}

}  // extern "C"

int gca::check_topk(const LmkTopkArgs* a) {
  if (!a) return GCA_ERR_NULL;
  if (!a->lmk_q || !a->lmk_k || !a->out_keys) return GCA_ERR_NULL;
  if (a->N < 0 || a->Cq < 0 || a->E < 0) return GCA_ERR_SHAPE;
  if (a->D < 8 || a->D % 8 != 0 || a->D > 1024 || a->K < 1 || a->K > 32) return GCA_ERR_SHAPE;
  if (a->head_dim != 0 && (a->head_dim != 64 || a->D % 64 != 0 || a->noise)) return GCA_ERR_SHAPE;
  if (!aligned16(a->lmk_q) || !aligned16(a->lmk_k)) return GCA_ERR_ALIGN;
  if (a->q_row_stride % 8 || a->k_row_stride % 8 || a->q_batch_stride % 8 || a->k_batch_stride % 8) return GCA_ERR_STRIDE;
  if (a->e_base < 0 || a->e_base + a->E >= 0xffffffffll) return GCA_ERR_TOO_LARGE;
  if (a->splits < 0) return GCA_ERR_SHAPE;
  return 0;
}

extern "C" {

size_t lmk_topk_workspace_bytes(const LmkTopkArgs* a) {
  if (gca::check_topk(a)) return 0;
  // A size query must not fail for lack of a device: when the landmark pointer cannot be
  // attributed to one, 256 SMs are assumed, which can only over-estimate (more SMs = more splits).
  gca::DeviceScope scope(a->lmk_k);
  return gca::lmk_topk_workspace_bytes_impl(*a, scope.rc ? 256 : gca::sm_count(scope.dev));
}

int lmk_score_topk(const LmkTopkArgs* a, void* stream) {
  int rc = gca::check_topk(a);
  if (rc) return rc;
  if (a->N == 0 || a->Cq == 0) return 0;
  if (!a->workspace) return GCA_ERR_WORKSPACE;
  gca::DeviceScope scope(a->lmk_k);
  if (scope.rc) return scope.rc;
  const int sms = gca::sm_count(scope.dev);
  const size_t need = gca::lmk_topk_workspace_bytes_impl(*a, sms);
  if (a->workspace_bytes < need) return GCA_ERR_WORKSPACE;
  return gca::launch_lmk_score_topk(*a, a->workspace, sms, (cudaStream_t)stream);
}

int lmk_topk_merge(const LmkMergeArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->keys || !a->out_keys) return GCA_ERR_NULL;
  if (a->R < 0 || a->P < 1 || a->K < 1 || a->K > 32) return GCA_ERR_SHAPE;
  if (a->R == 0) return 0;
  gca::DeviceScope scope(a->keys);
  if (scope.rc) return scope.rc;
  return gca::launch_lmk_merge(*a, (cudaStream_t)stream);
}

int gca_cache_append(const CacheAppendArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->new_k || !a->new_v || !a->k_cache || !a->v_cache) return GCA_ERR_NULL;
  const int es = esize_of(a->dtype);
  if (es == 0) return GCA_ERR_DTYPE;
  if (a->N < 0 || a->count < 0 || a->pos < 0 || a->L < 1 || a->HD < 1) return GCA_ERR_SHAPE;
  if ((a->HD * es) % 16 != 0 || (a->new_lmk && (a->Dm * es) % 16 != 0)) return GCA_ERR_SHAPE;
  if ((a->new_batch_stride * es) % 16 || (a->cache_batch_stride * es) % 16) return GCA_ERR_STRIDE;
  if (a->new_lmk && ((a->new_lmk_batch_stride * es) % 16 || (a->lmk_cache_batch_stride * es) % 16)) return GCA_ERR_STRIDE;
  if (!aligned16(a->new_k) || !aligned16(a->new_v) || !aligned16(a->k_cache) || !aligned16(a->v_cache)) return GCA_ERR_ALIGN;
  if (a->new_lmk && (!aligned16(a->new_lmk) || !a->lmk_cache || !aligned16(a->lmk_cache))) return GCA_ERR_ALIGN;
  // the destination must hold chunks pos .. pos + count - 1
  if ((long long)a->pos + a->count > a->capacity) return GCA_ERR_SHAPE;
  if (a->new_lmk && (long long)a->pos + a->count > a->lmk_capacity) return GCA_ERR_SHAPE;
  if (a->N == 0 || a->count == 0) return 0;
  gca::DeviceScope scope(a->k_cache);
  if (scope.rc) return scope.rc;
  return gca::launch_cache_append(*a, (cudaStream_t)stream);
}

int gca_kv_project_append(const KvProjectArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->x || !a->wk || !a->wv || !a->k_cache || !a->v_cache) return GCA_ERR_NULL;
  if (a->N < 0 || a->count < 0 || a->pos < 0 || a->D < 256 || a->D % 256 != 0) return GCA_ERR_SHAPE;
  if ((long long)a->pos + a->count > a->capacity) return GCA_ERR_SHAPE;
  if (a->lmk_cache && (long long)a->pos + a->count > a->lmk_capacity) return GCA_ERR_SHAPE;
  if (a->cache_batch_stride % 16 || (a->lmk_cache && a->lmk_cache_batch_stride % 8)) return GCA_ERR_STRIDE;
  if ((reinterpret_cast<uintptr_t>(a->k_cache) & 31u) || (reinterpret_cast<uintptr_t>(a->v_cache) & 31u) || !aligned16(a->x) ||
      !aligned16(a->wk) || !aligned16(a->wv) || (a->lmk_cache && !aligned16(a->lmk_cache)))
    return GCA_ERR_ALIGN;
  if ((long long)a->N * a->count * 64 >= (1ll << 31)) return GCA_ERR_TOO_LARGE;
  if (a->N == 0 || a->count == 0) return 0;
  gca::DeviceScope scope(a->k_cache);
  if (scope.rc) return scope.rc;
  return gca::launch_kv_project_append(*a, gca::sm_count(scope.dev), (cudaStream_t)stream);
}

int gca_row_rms(const RowRmsArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->x || !a->row_scale) return GCA_ERR_NULL;
  if (a->M < 0 || a->D < 8 || a->D % 8 != 0) return GCA_ERR_SHAPE;
  if (a->x_stride % 8 != 0 || a->x_stride < a->D) return GCA_ERR_STRIDE;
  if (!aligned16(a->x)) return GCA_ERR_ALIGN;
  if (a->M == 0) return 0;
  gca::DeviceScope scope(a->x);
  if (scope.rc) return scope.rc;
  return gca::launch_row_rms(*a, (cudaStream_t)stream);
}

int gca_silu_mul(const void* gate_up, void* out, int64_t M, int32_t I, int64_t in_stride, int64_t out_stride, void* stream) {
  if (!gate_up || !out) return GCA_ERR_NULL;
  if (M < 0 || I < 8 || I % 8 != 0) return GCA_ERR_SHAPE;
  if (in_stride % 8 != 0 || in_stride < 2 * (int64_t)I || out_stride % 8 != 0 || out_stride < I) return GCA_ERR_STRIDE;
  if (!aligned16(gate_up) || !aligned16(out)) return GCA_ERR_ALIGN;
  if (M == 0) return 0;
  gca::DeviceScope scope(out);
  if (scope.rc) return scope.rc;
  return gca::launch_silu_mul(gate_up, out, M, I, in_stride, out_stride, (cudaStream_t)stream);
}

size_t gca_linear_ce_workspace_bytes(int64_t M, int32_t N) {
  if (M <= 0 || N <= 0) return 0;
  const size_t tiles = ((size_t)N + 255) / 256;
  return gca::align_up((size_t)M * tiles * sizeof(float) * 2 + (size_t)M * sizeof(float), 256);
}

int gca_linear_cross_entropy(const LinearCeArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->x || !a->w || !a->targets || !a->loss) return GCA_ERR_NULL;
  if (a->M < 0 || a->N < 1 || a->K < 64 || a->K % 64 != 0) return GCA_ERR_SHAPE;
  if (a->x_stride % 8 || a->w_stride % 8 || a->x_stride < a->K || a->w_stride < a->K) return GCA_ERR_STRIDE;
  if (!aligned16(a->x) || !aligned16(a->w) || (reinterpret_cast<uintptr_t>(a->targets) & 7u)) return GCA_ERR_ALIGN;
  if (a->M == 0) return 0;
  if (!a->workspace || !aligned16(a->workspace)) return GCA_ERR_NULL;
  if ((size_t)a->workspace_bytes < gca_linear_ce_workspace_bytes(a->M, a->N)) return GCA_ERR_WORKSPACE;
  gca::DeviceScope scope(a->loss);
  if (scope.rc) return scope.rc;
  // a target outside [0, N) never gets its logit written: start from NaN so that the loss says so
  const size_t tiles = ((size_t)a->N + 255) / 256;
  cudaError_t e = cudaMemsetAsync(static_cast<char*>(a->workspace) + (size_t)a->M * tiles * sizeof(float) * 2, 0xFF,
                                  (size_t)a->M * sizeof(float), (cudaStream_t)stream);
  if (e != cudaSuccess) return (int)e;
  return gca::launch_linear_ce(*a, gca::sm_count(scope.dev), (cudaStream_t)stream);
}

int gca_window_shift_append(const WindowAppendArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->k_window || !a->v_window || !a->k_new || !a->v_new) return GCA_ERR_NULL;
  if (a->N < 0 || a->H <= 0 || a->T < 1 || a->T > 640) return GCA_ERR_SHAPE;
  for (int i = 0; i < 2; ++i)
    if (a->window_stride[i] % 8 || a->new_stride[i] % 8) return GCA_ERR_STRIDE;
  if (!aligned16(a->k_window) || !aligned16(a->v_window) || !aligned16(a->k_new) || !aligned16(a->v_new)) return GCA_ERR_ALIGN;
  if (a->N == 0) return 0;
  gca::DeviceScope scope(a->k_window);
  if (scope.rc) return scope.rc;
  return gca::launch_window_shift_append(*a, (cudaStream_t)stream);
}

static int check_window_decode(const WindowDecodeArgs* a) {
  if (!a->q || !a->k || !a->v || !a->out) return GCA_ERR_NULL;
  if (a->N < 0 || a->Hq <= 0 || a->Hkv <= 0 || a->Hq % a->Hkv || a->Sq <= 0 || a->T < a->Sq || a->window < 0) return GCA_ERR_SHAPE;
  if ((a->Hq / a->Hkv) * a->Sq > 4) return GCA_ERR_SHAPE;
  for (int i = 0; i < 3; ++i)
    if (a->q_stride[i] % 8 || a->o_stride[i] % 8 || a->k_stride[i] % 8 || a->v_stride[i] % 8) return GCA_ERR_STRIDE;
  if (!aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->out)) return GCA_ERR_ALIGN;
  return 0;
}

int gca_window_decode(const WindowDecodeArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (int rc = check_window_decode(a)) return rc;
  if (a->N == 0) return 0;
  gca::DeviceScope scope(a->out);
  if (scope.rc) return scope.rc;
  return gca::launch_window_decode(*a, (cudaStream_t)stream);
}

int gca_window_ring_decode(const WindowRingDecodeArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (int rc = check_window_decode(&a->attn)) return rc;
  if (!a->k_new || !a->v_new || !a->rows_written) return GCA_ERR_NULL;
  if (a->attn.Sq != 1 || a->attn.T > a->attn.window + 1) return GCA_ERR_SHAPE;   // every row of the ring is visible
  if (a->new_stride[0] % 8 || a->new_stride[1] % 8) return GCA_ERR_STRIDE;
  if (!aligned16(a->k_new) || !aligned16(a->v_new)) return GCA_ERR_ALIGN;
  if (a->attn.N == 0) return 0;
  gca::DeviceScope scope(a->attn.out);
  if (scope.rc) return scope.rc;
  return gca::launch_window_ring_decode(*a, (cudaStream_t)stream);
}

int gca_linear(const LinearArgs* a, void* stream) {
  if (!a) return GCA_ERR_NULL;
  if (!a->x || !a->w || !a->out) return GCA_ERR_NULL;
  if (a->M < 0 || a->N < 16 || a->N % 16 != 0 || a->K < 64 || a->K % 64 != 0) return GCA_ERR_SHAPE;
  if (a->x_stride % 8 || a->w_stride % 8 || a->out_stride % 8 || (a->residual && a->residual_stride % 8) ||
      a->x_stride < a->K || a->w_stride < a->K || a->out_stride < a->N || (a->residual && a->residual_stride < a->N))
    return GCA_ERR_STRIDE;
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->out) || (a->residual && !aligned16(a->residual))) return GCA_ERR_ALIGN;
  if (a->M == 0) return 0;
  gca::DeviceScope scope(a->out);
  if (scope.rc) return scope.rc;
  return gca::launch_linear(*a, gca::sm_count(scope.dev), (cudaStream_t)stream);
}

}  // extern "C"
