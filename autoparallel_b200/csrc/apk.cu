// Host side of libapk.so: argument checking, TMA descriptor encoding, kernel launches and the
// symmetric-memory allocator behind the C ABI declared in include/apk.h.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "../../include/apk.h"
#include "gemm_kernel.cuh"
#include "collectives_kernel.cuh"

namespace {

thread_local char g_err[512] = "";
std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_pair_launches{0};
std::atomic<uint64_t> g_pair_refusals{0};

constexpr int kMaxDevices = 64;
std::mutex g_mu;   // guards every per-device cache below (calls may come from any thread)

// Timeline buffer set by apk_set_trace (device memory of the device that was current then).
unsigned long long* g_trace = nullptr;
uint64_t g_trace_bytes = 0;
int g_trace_device = -1;

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

#define APK_CUDA(expr)                                                                          \
  do {                                                                                          \
    cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess) return fail(APK_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

using EncodeFn = PFN_cuTensorMapEncodeTiled_v12000;

// libcuda is reached through the runtime, so the library loads on machines without a driver.
int get_encode(EncodeFn* out) {
  static EncodeFn fn = nullptr;
  static std::mutex mu;
  std::lock_guard<std::mutex> lk(mu);
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    APK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
    if (q != cudaDriverEntryPointSuccess || p == nullptr) return fail(APK_ERR_CUDA, "cuTensorMapEncodeTiled not found");
    fn = reinterpret_cast<EncodeFn>(p);
  }
  *out = fn;
  return APK_OK;
}

// 2-D row-major tensor [rows][cols] with `ld` elements between rows, box [box_rows][box_cols],
// 128-byte swizzle, out-of-range reads give zeros.
int encode_2d(CUtensorMap* tm, int dtype, const void* base, uint64_t cols, uint64_t rows, uint64_t ld,
              uint32_t box_cols, uint32_t box_rows, const char* what) {
  EncodeFn enc;
  int rc = get_encode(&enc);
  if (rc != APK_OK) return rc;
  const uint64_t es = (dtype == APK_E4M3) ? 1 : 2;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return fail(APK_ERR_ARG, "%s: base pointer must be 16-byte aligned", what);
  if ((ld * es) % 16 != 0) return fail(APK_ERR_ARG, "%s: row pitch (%llu bytes) must be a multiple of 16", what, (unsigned long long)(ld * es));
  if (box_cols * es != apk::ROW_BYTES) return fail(APK_ERR_ARG, "%s: inner box must span 128 bytes", what);
  if (box_rows > 256) return fail(APK_ERR_ARG, "%s: box rows > 256", what);
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType tmt = dtype == APK_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                  : dtype == APK_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(tm, tmt, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(APK_ERR_CUDA, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return APK_OK;
}

struct DeviceInfo {
  int sms = 0;
  int clock_khz = 0;
  bool ok = false;
};

int device_info(DeviceInfo* out) {
  static DeviceInfo cache[kMaxDevices];
  int dev = 0;
  APK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(APK_ERR_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_mu);
  if (!cache[dev].ok) {
    int major = 0;
    APK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
    if (major != 10) return fail(APK_ERR_CUDA, "device %d has compute capability %d.x; this library needs sm_100", dev, major);
    APK_CUDA(cudaDeviceGetAttribute(&cache[dev].sms, cudaDevAttrMultiProcessorCount, dev));
    APK_CUDA(cudaDeviceGetAttribute(&cache[dev].clock_khz, cudaDevAttrClockRate, dev));
    cache[dev].ok = true;
  }
  *out = cache[dev];
  return APK_OK;
}

// Why a device cannot run CTA pairs (empty: it can, or nobody has tried yet). Set once per device, and only
// when the occupancy query or the launch itself says that clusters of two are not schedulable.
char g_pair_unsupported[kMaxDevices][160] = {};

template <int BN, int STAGES, bool FP8, bool PAIR, bool TRACE>
int launch_instance_t(apk::KParams kp, long long units, const DeviceInfo& di, cudaStream_t stream) {
  using L = apk::SmemLayout<BN, STAGES, PAIR>;
  auto kern = apk::gemm_fused_kernel<BN, STAGES, FP8, PAIR, TRACE>;
  static bool configured[kMaxDevices] = {};
  static int max_clusters[kMaxDevices] = {};
  int dev = 0;
  APK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(APK_ERR_ARG, "device index %d out of range", dev);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(apk::NUM_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  // Cooperative whenever the group has peers: all CTAs must be resident at once, because the
  // communication warps of every CTA feed row blocks that other CTAs' producers wait for. With a
  // group of one no CTA waits for another (the two CTAs of a pair are co-scheduled by the cluster
  // launch itself), so a plain launch does.
  cudaLaunchAttribute attr[2];
  int na = 0;
  if (kp.ws > 1) {
    attr[na].id = cudaLaunchAttributeCooperative;
    attr[na].val.cooperative = 1;
    ++na;
  }
  {
    std::lock_guard<std::mutex> lk(g_mu);
    if (!configured[dev]) {
      APK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
      configured[dev] = true;
    }
    if (PAIR) {
      attr[na].id = cudaLaunchAttributeClusterDimension;
      attr[na].val.clusterDim.x = 2;
      attr[na].val.clusterDim.y = 1;
      attr[na].val.clusterDim.z = 1;
      ++na;
      cfg.attrs = attr;
      cfg.numAttrs = na;
      if (max_clusters[dev] == 0) {
        cfg.gridDim = dim3((unsigned)(di.sms & ~1));
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        if (e != cudaSuccess || n < 1) {
          cudaGetLastError();
          snprintf(g_pair_unsupported[dev], sizeof(g_pair_unsupported[dev]), "cudaOccupancyMaxActiveClusters: %s, %d clusters",
                   cudaGetErrorString(e), n);
          return fail(APK_ERR_CUDA, "CTA pairs cannot be scheduled on device %d (%s)", dev, g_pair_unsupported[dev]);
        }
        max_clusters[dev] = n;
        if (getenv("APK_VERBOSE") != nullptr) fprintf(stderr, "[apk] device %d: %d SMs, at most %d co-resident CTA pairs\n", dev, di.sms, n);
      }
    }
  }
  cfg.attrs = attr;
  cfg.numAttrs = na;
  if (PAIR) {
    const long long clusters = units < max_clusters[dev] ? units : max_clusters[dev];
    cfg.gridDim = dim3((unsigned)(2 * clusters));
  } else {
    cfg.gridDim = dim3((unsigned)(units < di.sms ? units : di.sms));
  }
  // Timeline: one record per (CTA, local tile), only when the buffer set by apk_set_trace is large enough.
  kp.trace = nullptr;
  kp.trace_tiles = 0;
  if (TRACE && g_trace != nullptr && g_trace_device == dev) {
    const long long sched_ctas = PAIR ? cfg.gridDim.x / 2 : cfg.gridDim.x;
    const long long per_cta = (units + sched_ctas - 1) / sched_ctas;
    const uint64_t need = (uint64_t)cfg.gridDim.x * (uint64_t)per_cta * apk::TRACE_FIELDS * 8;
    if (need <= g_trace_bytes) {
      kp.trace = g_trace;
      kp.trace_tiles = (int32_t)per_cta;
    }
  }
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, kp);
  if (e != cudaSuccess) {
    cudaGetLastError();
    if (PAIR && (e == cudaErrorCooperativeLaunchTooLarge || e == cudaErrorNotSupported || e == cudaErrorInvalidClusterSize)) {
      std::lock_guard<std::mutex> lk(g_mu);
      snprintf(g_pair_unsupported[dev], sizeof(g_pair_unsupported[dev]), "cluster launch: %s", cudaGetErrorString(e));
    }
    return fail(APK_ERR_CUDA, "launch of gemm_fused_kernel<%d,%d,%d,%d>: %s", BN, STAGES, (int)FP8, (int)PAIR, cudaGetErrorString(e));
  }
  g_launches.fetch_add(1);
  if (PAIR) g_pair_launches.fetch_add(1);
  return APK_OK;
}

// The instances with the timeline compiled in are used only while a timeline buffer is set for this device.
template <int BN, int STAGES, bool FP8, bool PAIR>
int launch_instance(const apk::KParams& kp, long long units, const DeviceInfo& di, cudaStream_t stream) {
  int dev = -1;
  cudaGetDevice(&dev);
  bool tracing;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    tracing = g_trace != nullptr && g_trace_device == dev;
  }
  return tracing ? launch_instance_t<BN, STAGES, FP8, PAIR, true>(kp, units, di, stream)
                 : launch_instance_t<BN, STAGES, FP8, PAIR, false>(kp, units, di, stream);
}

// CTA pairs (cta_group::2) are used when every output is a whole number of 256-column tiles and every
// chunk a whole number of 256-row tile pairs; APK_PAIR=0 in the environment turns them off.
bool pair_eligible(const apk::KParams& kp) {
  static std::once_flag once;
  static bool env_on = true;
  std::call_once(once, [] {
    const char* e = getenv("APK_PAIR");
    env_on = !(e != nullptr && e[0] == '0');
  });
  if (!env_on) return false;
  for (int b = 0; b < kp.nB; ++b) {
    if (kp.N[b] % 256 != 0) return false;
  }
  const long long mt = (kp.rows_per_rank + apk::BM - 1) / apk::BM;
  return mt % 2 == 0;
}

// Reduce-scatter: how many row blocks the own tiles trail the peers' (KParams::rs_lag). A peer's partial for
// row block j must be there before the owner's epilogue asks for it (measured at 8 ranks: acknowledged about
// 10 us after it was sent, announced about 8 us later; a tile takes about 14 us), so row block j of the own chunk
// follows about three grid waves behind the peers' row block j, and never less than the default of four row
// blocks. Not more than that: while only peers' tiles are computed every CTA sends 64 KiB per tile (about
// 780 GB/s per GPU, more than the fabric gives when all GPUs send) and at the end, when only own tiles are left,
// NVLink idles, so a longer lag costs on both ends (swept at 4 ranks: 12 row blocks 1.216 ms per step, 5: 1.207,
// 3: 1.188, same call).
int rs_lag_for(const apk::KParams& kp, long long nt, long long sched_ctas) {
  static std::once_flag once;
  static int forced = 0;     // APK_RS_LAG=<row blocks> in the environment overrides the rule below (tuning)
  std::call_once(once, [] {
    const char* e = getenv("APK_RS_LAG");
    if (e != nullptr && atoi(e) > 0) forced = atoi(e);
  });
  if (forced > 0) return forced;
  const long long per_row_block = nt * (kp.ws - 1);   // peers' units per row block
  if (per_row_block <= 0) return apk::RS_LAG;
  const long long want = (3 * sched_ctas + per_row_block - 1) / per_row_block;
  return (int)(want > apk::RS_LAG ? want : apk::RS_LAG);
}

int launch(const apk::KParams& kp_in, int max_n, bool fp8, cudaStream_t stream) {
  apk::KParams kp = kp_in;
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != APK_OK) return rc;
  const bool narrow = max_n <= 128;
  const int bn = narrow ? 128 : 256;
  long long nt = 0;
  for (int b = 0; b < kp.nB; ++b) nt += (kp.N[b] + bn - 1) / bn;
  const long long mt = (kp.rows_per_rank + apk::BM - 1) / apk::BM;
  const long long chunks = (kp.mode == apk::MODE_PLAIN || kp.ag_ksplit) ? 1 : kp.ws;
  const long long tiles = nt * mt * chunks;
  if (tiles <= 0) return APK_OK;
  if (tiles > 0x7fffffffLL) return fail(APK_ERR_ARG, "too many tiles");
  int dev = 0;
  APK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(APK_ERR_ARG, "device index %d out of range", dev);
  bool pair_ok;
  {
    std::lock_guard<std::mutex> lk(g_mu);
    pair_ok = g_pair_unsupported[dev][0] == '\0';
  }
  if (kp.mode == apk::MODE_RS && kp.ws > 1) kp.rs_lag = rs_lag_for(kp, nt, di.sms);
  if (!narrow && pair_eligible(kp)) {
    if (pair_ok) {
      if (kp.mode == apk::MODE_RS && kp.ws > 1) kp.rs_lag = rs_lag_for(kp, nt, di.sms / 2);
      rc = fp8 ? launch_instance<256, 6, true, true>(kp, tiles / 2, di, stream)
               : launch_instance<256, 6, false, true>(kp, tiles / 2, di, stream);
      bool unsupported;
      {
        std::lock_guard<std::mutex> lk(g_mu);
        unsupported = g_pair_unsupported[dev][0] != '\0';
      }
      if (rc == APK_OK || !unsupported) return rc;   // any other failure is the caller's to see
    }
    g_pair_refusals.fetch_add(1);   // this device cannot run pairs: single CTAs, and the count says so
    if (kp.mode == apk::MODE_RS && kp.ws > 1) kp.rs_lag = rs_lag_for(kp, nt, di.sms);
  }
  if (narrow) {
    return fp8 ? launch_instance<128, 6, true, false>(kp, tiles, di, stream) : launch_instance<128, 6, false, false>(kp, tiles, di, stream);
  }
  return fp8 ? launch_instance<256, 4, true, false>(kp, tiles, di, stream) : launch_instance<256, 4, false, false>(kp, tiles, di, stream);
}

uint64_t align_up(uint64_t x, uint64_t a) { return (x + a - 1) / a * a; }

int fill_operand(apk::KParams* kp, int b, const apk_operand& op_in, int dtype, int K, int bn, int64_t out_rows, const char* what,
                 int b_cols_total = 0) {
  // b_cols_total: columns of the B tensor when the op works on a column slice of it (op.N is the slice width)
  apk_operand op = op_in;
  const uint64_t b_cols = b_cols_total > 0 ? (uint64_t)b_cols_total : (uint64_t)op.N;
  if (op.B == nullptr || op.out == nullptr) return fail(APK_ERR_ARG, "%s: null B or out", what);
  if (op.N <= 0) return fail(APK_ERR_ARG, "%s: N must be positive", what);
  if (op.out_dtype != APK_BF16 && op.out_dtype != APK_F32 && op.out_dtype != APK_F16)
    return fail(APK_ERR_ARG, "%s: out dtype must be bf16, f16 or f32", what);
  const int oes = op.out_dtype == APK_F32 ? 4 : 2;
  const int vec = 16 / oes;
  if (op.N % vec != 0) return fail(APK_ERR_ARG, "%s: N (%d) must be a multiple of %d", what, op.N, vec);
  if ((reinterpret_cast<uintptr_t>(op.out) & 15u) != 0 || (op.ldo * oes) % 16 != 0)
    return fail(APK_ERR_ARG, "%s: output must be 16-byte aligned with a 16-byte multiple pitch", what);
  const int bke = dtype == APK_E4M3 ? 128 : 64;
  int rc;
  if (op.n_major) {
    rc = encode_2d(&kp->tmB[b], dtype, op.B, b_cols, (uint64_t)K, (uint64_t)op.ldb, bke, bke, what);
  } else {
    rc = encode_2d(&kp->tmB[b], dtype, op.B, (uint64_t)K, b_cols, (uint64_t)op.ldb, bke, bn, what);
    if (rc == APK_OK && bn == 256)   // a CTA of a pair loads 128 of the tile's 256 columns
      rc = encode_2d(&kp->tmBp[b], dtype, op.B, (uint64_t)K, b_cols, (uint64_t)op.ldb, bke, bn / 2, what);
  }
  if (rc != APK_OK) return rc;
  kp->N[b] = op.N;
  kp->b_nmajor[b] = op.n_major ? 1 : 0;
  kp->out[b] = op.out;
  kp->ldo[b] = op.ldo;
  kp->out_fp32[b] = op.out_dtype == APK_F32;
  kp->out_f16[b] = op.out_dtype == APK_F16;
  if (op.out_dtype != APK_F32) {
    // stores: 32 rows x 64 columns per TMA instruction, clipped at N by the descriptor
    rc = encode_2d(&kp->tmOut[b], op.out_dtype, op.out, (uint64_t)op.N, (uint64_t)out_rows, (uint64_t)op.ldo, 64, 32, what);
    if (rc != APK_OK) return rc;
    kp->out_tma[b] = 1;
  }
  if (op.b_scale_mode != APK_SCALE_NONE && op.b_scale_mode != APK_SCALE_SCALAR && op.b_scale_mode != APK_SCALE_VECTOR)
    return fail(APK_ERR_ARG, "%s: bad b_scale_mode", what);
  if (op.b_scale_mode != APK_SCALE_NONE && op.b_scale == nullptr) return fail(APK_ERR_ARG, "%s: b_scale is null", what);
  kp->b_scale[b] = op.b_scale;
  kp->b_scale_mode[b] = op.b_scale_mode;
  kp->bias[b] = op.bias;
  kp->bias_fp32[b] = op.bias_dtype == APK_F32;
  kp->result_scale[b] = op.result_scale;
  return APK_OK;
}

int check_comm(const apk_comm* c) {
  if (c == nullptr) return fail(APK_ERR_ARG, "comm is null");
  if (c->world < 1 || c->world > APK_MAX_WORLD) return fail(APK_ERR_ARG, "world must be in [1, %d]", APK_MAX_WORLD);
  if (c->rank < 0 || c->rank >= c->world) return fail(APK_ERR_ARG, "rank out of range");
  if (c->status == nullptr) return fail(APK_ERR_ARG, "comm.status is null");
  if (c->world > 1) {
    for (int r = 0; r < c->world; ++r) {
      if (c->data[r] == nullptr || c->flags[r] == nullptr) return fail(APK_ERR_ARG, "comm.data/flags[%d] is null", r);
    }
    if (c->flag_bytes < 8192) return fail(APK_ERR_SIZE, "signal pad too small");
    if (c->ctrl == nullptr) return fail(APK_ERR_ARG, "comm.ctrl is null");
  }
  return APK_OK;
}

long long timeout_cycles(const apk_comm* c, const DeviceInfo& di) {
  double s = c->timeout_s > 0 ? c->timeout_s : 30.0;
  return (long long)(s * 1e3 * (double)di.clock_khz);
}

constexpr uint64_t kFlagRsOffset = 4096;  // bytes: staged flags live below, per-tile flags above

}  // namespace

// The order in which one CTA (or CTA pair) enumeration visits the tiles, computed on the host with the
// very functions the kernel uses. For tests of the schedule; needs no GPU.
template <int BN, bool PAIR>
int schedule_rows(const apk::KParams& kp, int crank, int32_t* out, int capacity) {
  const apk::Sched sc = apk::make_sched<BN, PAIR>(kp);
  if (out != nullptr) {
    for (int t = 0; t < sc.total_tiles && t < capacity; ++t) {
      const apk::TileInfo ti = apk::decode_tile<BN, PAIR>(kp, sc, t, crank);
      int32_t* r = out + 6 * (size_t)t;
      r[0] = ti.chunk; r[1] = ti.mt; r[2] = ti.b; r[3] = ti.n0; r[4] = ti.tile_in_chunk; r[5] = ti.rows_valid;
    }
  }
  return sc.total_tiles;
}

extern "C" {

int apk_abi_version(void) { return APK_ABI_VERSION; }
const char* apk_last_error(void) { return g_err; }
uint64_t apk_launch_count(void) { return g_launches.load(); }
uint64_t apk_pair_launch_count(void) { return g_pair_launches.load(); }
uint64_t apk_pair_refusal_count(void) { return g_pair_refusals.load(); }

int apk_set_trace(void* buf, uint64_t bytes) {
  int dev = 0;
  APK_CUDA(cudaGetDevice(&dev));
  if (buf != nullptr && (reinterpret_cast<uintptr_t>(buf) & 7u) != 0) return fail(APK_ERR_ARG, "apk_set_trace: buffer must be 8-byte aligned");
  std::lock_guard<std::mutex> lk(g_mu);
  g_trace = reinterpret_cast<unsigned long long*>(buf);
  g_trace_bytes = buf != nullptr ? bytes : 0;
  g_trace_device = buf != nullptr ? dev : -1;
  return APK_OK;
}

int apk_symm_alloc(uint64_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) return fail(APK_ERR_ARG, "apk_symm_alloc: bad arguments");
  void* p = nullptr;
  APK_CUDA(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(APK_ERR_CUDA, "cudaMemset: %s", cudaGetErrorString(e));
  }
  APK_CUDA(cudaDeviceSynchronize());
  *ptr = p;
  return APK_OK;
}

int apk_symm_free(void* ptr) {
  if (ptr == nullptr) return APK_OK;
  APK_CUDA(cudaFree(ptr));
  return APK_OK;
}

int apk_symm_export(const void* ptr, uint8_t handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle is 64 bytes");
  if (ptr == nullptr || handle == nullptr) return fail(APK_ERR_ARG, "apk_symm_export: null argument");
  cudaIpcMemHandle_t h;
  APK_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
  memcpy(handle, &h, 64);
  return APK_OK;
}

int apk_symm_import(const uint8_t handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return fail(APK_ERR_ARG, "apk_symm_import: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  APK_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return APK_OK;
}

int apk_symm_unimport(void* ptr) {
  if (ptr == nullptr) return APK_OK;
  APK_CUDA(cudaIpcCloseMemHandle(ptr));
  return APK_OK;
}

uint64_t apk_ag_gemm_arena_bytes(const apk_ag_gemm_args* a, int32_t world) {
  if (a == nullptr || world <= 1) return 0;
  const uint64_t es = a->dtype == APK_E4M3 ? 1 : 2;
  uint64_t bytes = align_up((uint64_t)a->rows_per_rank * (uint64_t)a->K * es, 256);
  if (a->a_scale_mode == APK_SCALE_VECTOR) bytes += align_up((uint64_t)a->rows_per_rank * 4, 256);
  return bytes;
}

uint64_t apk_gemm_rs_arena_bytes(const apk_gemm_rs_args* a, int32_t world) {
  if (a == nullptr || world <= 1) return 0;
  const uint64_t rows = a->scatter_cols ? (uint64_t)a->M : (uint64_t)(a->M / world);   // rows of one destination's part
  const uint64_t width = a->scatter_cols ? (uint64_t)(a->B.N / world) : (uint64_t)a->B.N;
  const uint64_t mt = (rows + apk::BM - 1) / apk::BM;
  if (a->B.out_dtype == APK_F32) {
    // fp32 partials: row-major, one slot per source rank padded to whole 128-row tiles
    return align_up((uint64_t)world * mt * apk::BM * width * 4, 256);
  }
  // bf16 partials: whole tiles, stored as contiguous 32 x 64 blocks
  const uint64_t bn = width <= 128 ? 128 : 256;
  const uint64_t nt = (width + bn - 1) / bn;
  // one slot per source rank, plus the fp32 sums of the peers' partials (twice a slot)
  return (uint64_t)(world + 2) * mt * nt * apk::BM * bn * 2;
}

uint64_t apk_ctrl_bytes(int32_t rows_per_rank, int32_t world) {
  const uint64_t mt = ((uint64_t)rows_per_rank + apk::BM - 1) / apk::BM;
  return 256 + 4 * mt * (uint64_t)(world < 1 ? 1 : world);
}

int apk_ag_gemm(const apk_comm* comm, const apk_ag_gemm_args* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = check_comm(comm);
  if (rc != APK_OK) return rc;
  if (a == nullptr) return fail(APK_ERR_ARG, "args is null");
  if (a->dtype != APK_BF16 && a->dtype != APK_E4M3 && a->dtype != APK_F16) return fail(APK_ERR_ARG, "dtype must be bf16, f16 or e4m3");
  if (a->nB < 1 || a->nB > APK_MAX_B) return fail(APK_ERR_ARG, "nB must be in [1, %d]", APK_MAX_B);
  if (a->rows_per_rank < 0 || a->K <= 0) return fail(APK_ERR_ARG, "bad shape");
  if (a->rows_per_rank == 0) return APK_OK;
  if (a->A_shard == nullptr) return fail(APK_ERR_ARG, "A_shard is null");
  const int ws = comm->world;
  const int es = a->dtype == APK_E4M3 ? 1 : 2;
  const int64_t M = (int64_t)a->rows_per_rank * ws;
  if (M > 0x7fffffffLL) return fail(APK_ERR_ARG, "M too large");
  const bool need_gathered = ws > 1 || a->return_A;
  if (need_gathered && a->A_gathered == nullptr) return fail(APK_ERR_ARG, "A_gathered is required");
  if (((int64_t)a->K * es) % 16 != 0) return fail(APK_ERR_ARG, "K * element size must be a multiple of 16 bytes");
  DeviceInfo di;
  rc = device_info(&di);
  if (rc != APK_OK) return rc;

  apk::KParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.mode = apk::MODE_AG;
  kp.ws = ws;
  kp.rank = comm->rank;
  kp.nB = a->nB;
  kp.M = (int32_t)M;
  kp.K = a->K;
  kp.ag_ksplit = a->gather_k ? 1 : 0;
  if (a->gather_k && (a->dtype == APK_E4M3 || a->a_scale_mode != APK_SCALE_NONE))
    return fail(APK_ERR_ARG, "gather_k supports bf16 / f16 without scales only");
  if (a->gather_k && (int64_t)a->K * ws > 0x7fffffffLL) return fail(APK_ERR_ARG, "K too large");
  // K-split: a k-block that runs past a shard's K would multiply A's zero fill with the NEXT rank's rows of B
  // (0 * Inf = NaN where the reference's cat(A) @ B has none), so every slice must be whole k-blocks.
  if (a->gather_k && ws > 1 && a->K % 64 != 0) return fail(APK_ERR_ARG, "gather_k needs K (%d) to be a multiple of 64", a->K);
  kp.rows_per_rank = a->rows_per_rank;
  kp.elem_bytes = es;
  kp.in_f16 = a->dtype == APK_F16;
  int max_n = 0;
  for (int b = 0; b < a->nB; ++b) max_n = a->Bs[b].N > max_n ? a->Bs[b].N : max_n;
  const int bn = max_n <= 128 ? 128 : 256;
  const int bke = a->dtype == APK_E4M3 ? 128 : 64;
  rc = encode_2d(&kp.tmA0, a->dtype, a->A_shard, (uint64_t)a->K, (uint64_t)a->rows_per_rank, (uint64_t)a->lda, bke, apk::BM, "A_shard");
  if (rc != APK_OK) return rc;
  if (need_gathered) {
    rc = encode_2d(&kp.tmA1, a->dtype, a->A_gathered, (uint64_t)a->K, (uint64_t)M, (uint64_t)a->K, bke, apk::BM, "A_gathered");
    if (rc != APK_OK) return rc;
  }
  for (int b = 0; b < a->nB; ++b) {
    // K-split: B spans all ranks' K-slices and the outputs have the shard's rows only
    rc = fill_operand(&kp, b, a->Bs[b], a->dtype, a->gather_k ? a->K * ws : a->K, bn, a->gather_k ? a->rows_per_rank : M, "Bs[i]");
    if (rc != APK_OK) return rc;
  }
  // A scale
  switch (a->a_scale_mode) {
    case APK_SCALE_NONE:
      break;
    case APK_SCALE_SCALAR:
      kp.a_scale_mode = 1;
      kp.a_scale_full = a->A_scale;
      break;
    case APK_SCALE_VECTOR:
      kp.a_scale_mode = 2;
      kp.a_scale_own = a->A_scale;
      if (ws > 1 && a->A_scale_gathered == nullptr) return fail(APK_ERR_ARG, "A_scale_gathered is required");
      kp.ag_has_scale = ws > 1;
      kp.ag_scale_src = a->A_scale;
      kp.ag_scale_gathered = a->A_scale_gathered;
      break;
    case APK_SCALE_ROWS_REPLICATED:
      kp.a_scale_mode = 2;
      kp.a_scale_full = a->A_scale;
      break;
    default:
      return fail(APK_ERR_ARG, "bad a_scale_mode");
  }
  if (a->a_scale_mode != APK_SCALE_NONE && a->A_scale == nullptr) return fail(APK_ERR_ARG, "A_scale is null");

  kp.ag_src = reinterpret_cast<const uint8_t*>(a->A_shard);
  kp.ag_chunk_bytes = (int64_t)a->rows_per_rank * a->K * es;
  kp.ag_gathered = reinterpret_cast<uint8_t*>(a->A_gathered);
  kp.ag_copy_own = a->return_A ? 1 : 0;
  if ((ws > 1 || a->return_A) && a->lda != a->K) return fail(APK_ERR_ARG, "A_shard must be contiguous (lda == K)");
  kp.ag_scale_off = (int64_t)align_up((uint64_t)kp.ag_chunk_bytes, 256);
  kp.epoch = comm->epoch;
  kp.status = comm->status;
  kp.timeout_cycles = timeout_cycles(comm, di);
  kp.reduce_scale = 1.0f;
  const uint64_t ctrl_need = apk_ctrl_bytes(a->rows_per_rank, ws);
  if (ws > 1) {
    const uint64_t half = comm->data_bytes / 2;
    const uint64_t need = apk_ag_gemm_arena_bytes(a, ws);
    if (need > half) return fail(APK_ERR_SIZE, "all-gather staging needs %llu bytes per half, arena has %llu", (unsigned long long)need, (unsigned long long)half);
    if (ctrl_need > comm->ctrl_bytes) return fail(APK_ERR_SIZE, "ctrl scratch too small");
    const uint64_t off = (comm->epoch & 1u) ? half : 0;
    for (int r = 0; r < ws; ++r) {
      kp.ag_symm_peer[r] = reinterpret_cast<const uint8_t*>(comm->data[r]) + off;
      kp.staged_peer[r] = reinterpret_cast<uint32_t*>(comm->flags[r]);
    }
    kp.ag_symm_local = reinterpret_cast<uint8_t*>(comm->data[comm->rank]) + off;
    kp.staged_local = reinterpret_cast<uint32_t*>(comm->flags[comm->rank]);
    kp.ctrl = reinterpret_cast<uint32_t*>(comm->ctrl);
    kp.ready = kp.ctrl + 64;
    APK_CUDA(cudaMemsetAsync(comm->ctrl, 0, ctrl_need, stream));
  }
  return launch(kp, max_n, a->dtype == APK_E4M3, stream);
}

int apk_gemm_rs(const apk_comm* comm, const apk_gemm_rs_args* a, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  int rc = check_comm(comm);
  if (rc != APK_OK) return rc;
  if (a == nullptr) return fail(APK_ERR_ARG, "args is null");
  if (a->dtype != APK_BF16 && a->dtype != APK_E4M3 && a->dtype != APK_F16) return fail(APK_ERR_ARG, "dtype must be bf16, f16 or e4m3");
  const int ws = comm->world;
  if (a->M < 0 || a->K <= 0) return fail(APK_ERR_ARG, "bad shape");
  if (!a->scatter_cols && a->M % ws != 0) return fail(APK_ERR_ARG, "M (%d) must be divisible by the group size (%d)", a->M, ws);
  if (a->scatter_cols && (a->B.N % ws != 0 || a->a_scale_mode != APK_SCALE_NONE || a->B.b_scale_mode != APK_SCALE_NONE))
    return fail(APK_ERR_ARG, "scatter_cols needs N divisible by the group size and no scales");
  if (a->M == 0) return APK_OK;
  if (a->A == nullptr) return fail(APK_ERR_ARG, "A is null");
  if (a->reduce_op != APK_REDUCE_SUM && a->reduce_op != APK_REDUCE_AVG) return fail(APK_ERR_ARG, "reduce_op must be sum or avg");
  const int es = a->dtype == APK_E4M3 ? 1 : 2;
  if (((int64_t)a->K * es) % 16 != 0) return fail(APK_ERR_ARG, "K * element size must be a multiple of 16 bytes");
  DeviceInfo di;
  rc = device_info(&di);
  if (rc != APK_OK) return rc;

  apk::KParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.mode = apk::MODE_RS;
  kp.ws = ws;
  kp.rank = comm->rank;
  kp.nB = 1;
  kp.M = a->M;
  kp.K = a->K;
  kp.rs_colsplit = a->scatter_cols ? 1 : 0;
  kp.rows_per_rank = a->scatter_cols ? a->M : a->M / ws;
  const int width = a->scatter_cols ? a->B.N / ws : a->B.N;   // columns of one destination's part
  kp.rs_slot_rows = (int32_t)align_up((uint64_t)kp.rows_per_rank, apk::BM);
  kp.elem_bytes = es;
  kp.in_f16 = a->dtype == APK_F16;
  if (ws > 1 && a->B.out_dtype == APK_F16)
    return fail(APK_ERR_ARG, "reduce-scatter partials travel as bf16 or f32: with peers, ask for an f32 output and round it to f16 afterwards");
  const int bn = width <= 128 ? 128 : 256;
  const int bke = a->dtype == APK_E4M3 ? 128 : 64;
  rc = encode_2d(&kp.tmA0, a->dtype, a->A, (uint64_t)a->K, (uint64_t)a->M, (uint64_t)a->lda, bke, apk::BM, "A");
  if (rc != APK_OK) return rc;
  {
    apk_operand opB = a->B;
    opB.N = width;
    rc = fill_operand(&kp, 0, opB, a->dtype, a->K, bn, kp.rows_per_rank, "B", a->B.N);
  }
  if (rc != APK_OK) return rc;
  switch (a->a_scale_mode) {
    case APK_SCALE_NONE:
      break;
    case APK_SCALE_SCALAR:
      kp.a_scale_mode = 1;
      kp.a_scale_full = a->A_scale;
      break;
    case APK_SCALE_VECTOR:
    case APK_SCALE_ROWS_REPLICATED:
      kp.a_scale_mode = 2;
      kp.a_scale_full = a->A_scale;
      break;
    default:
      return fail(APK_ERR_ARG, "bad a_scale_mode");
  }
  if (a->a_scale_mode != APK_SCALE_NONE && a->A_scale == nullptr) return fail(APK_ERR_ARG, "A_scale is null");
  kp.reduce_scale = a->reduce_op == APK_REDUCE_AVG ? 1.0f / (float)ws : 1.0f;
  kp.epoch = comm->epoch;
  kp.status = comm->status;
  kp.timeout_cycles = timeout_cycles(comm, di);
  if (ws > 1) {
    const uint64_t half = comm->data_bytes / 2;
    const uint64_t need = apk_gemm_rs_arena_bytes(a, ws);
    if (need > half) return fail(APK_ERR_SIZE, "reduce-scatter arena needs %llu bytes per half, arena has %llu", (unsigned long long)need, (unsigned long long)half);
    const uint64_t max_tiles = (comm->flag_bytes - kFlagRsOffset) / 4 / (uint64_t)ws;
    const uint64_t tiles = (uint64_t)((kp.rows_per_rank + apk::BM - 1) / apk::BM) * (uint64_t)((width + bn - 1) / bn);
    if (tiles > max_tiles) return fail(APK_ERR_SIZE, "signal pad holds %llu tile flags per rank, need %llu", (unsigned long long)max_tiles, (unsigned long long)tiles);
    kp.rs_max_tiles = (int32_t)max_tiles;
    kp.rs_slot_rows = (int32_t)align_up((uint64_t)kp.rows_per_rank, apk::BM);
    const uint64_t off = (comm->epoch & 1u) ? half : 0;
    if ((half & 15u) != 0) return fail(APK_ERR_ARG, "arena halves must be 16-byte aligned");
    for (int r = 0; r < ws; ++r) {
      kp.rs_arena_peer[r] = reinterpret_cast<uint8_t*>(comm->data[r]) + off;
      kp.rs_flag_peer[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(comm->flags[r]) + kFlagRsOffset);
    }
    kp.rs_arena_tma = a->B.out_dtype == APK_BF16;
    kp.rs_arena_local = kp.rs_arena_peer[comm->rank];
    kp.rs_sum_local = reinterpret_cast<float*>(kp.rs_arena_local + (uint64_t)ws * tiles * apk::BM * bn * 2);
    kp.rs_flag_local = kp.rs_flag_peer[comm->rank];
  }
  return launch(kp, width, a->dtype == APK_E4M3, stream);
}

// ---- stand-alone collectives over the same arena / flags / epoch protocol
static int coll_common(const apk_comm* comm, uint64_t chunk_bytes, uint64_t arena_need, apk::CParams* cp, cudaStream_t stream) {
  int rc = check_comm(comm);
  if (rc != APK_OK) return rc;
  if (chunk_bytes % 16 != 0) return fail(APK_ERR_ARG, "every rank's part (%llu bytes) must be a multiple of 16 bytes", (unsigned long long)chunk_bytes);
  DeviceInfo di;
  rc = device_info(&di);
  if (rc != APK_OK) return rc;
  memset(cp, 0, sizeof(*cp));
  cp->ws = comm->world;
  cp->rank = comm->rank;
  cp->epoch = comm->epoch;
  cp->chunk_bytes = (long long)chunk_bytes;
  cp->status = comm->status;
  cp->timeout_cycles = timeout_cycles(comm, di);
  cp->reduce_scale = 1.0f;
  if (comm->world > 1) {
    const uint64_t half = comm->data_bytes / 2;
    if (arena_need > half) return fail(APK_ERR_SIZE, "collective needs %llu bytes per arena half, arena has %llu", (unsigned long long)arena_need, (unsigned long long)half);
    const uint64_t off = (comm->epoch & 1u) ? half : 0;
    for (int r = 0; r < comm->world; ++r) cp->symm_peer[r] = reinterpret_cast<uint8_t*>(comm->data[r]) + off;
    cp->symm_local = cp->symm_peer[comm->rank];
    cp->ctrl = reinterpret_cast<uint32_t*>(comm->ctrl);
    APK_CUDA(cudaMemsetAsync(comm->ctrl, 0, 256, stream));
  }
  return APK_OK;
}

// Both collectives release the peers' flags only after a grid-wide count is complete while resident CTAs
// already spin on the peers' flags, so all CTAs must be co-resident: cooperative launch whenever there are
// peers, one CTA per SM (the occupancy query caps the grid if the device offers fewer slots).
static int launch_collective(void (*kern)(const apk::CParams), const apk::CParams& cp, cudaStream_t stream) {
  DeviceInfo di;
  int rc = device_info(&di);
  if (rc != APK_OK) return rc;
  int per_sm = 0;
  APK_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, apk::COLL_THREADS, 0));
  if (per_sm < 1) return fail(APK_ERR_CUDA, "the collective kernel does not fit on an SM");
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)di.sms);
  cfg.blockDim = dim3(apk::COLL_THREADS);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cp.ws > 1 ? 1 : 0;
  APK_CUDA(cudaLaunchKernelEx(&cfg, kern, cp));
  g_launches.fetch_add(1);
  return APK_OK;
}

int apk_all_gather(const apk_comm* comm, const void* shard, void* out, uint64_t shard_bytes, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (shard_bytes == 0) return APK_OK;
  if (shard == nullptr || out == nullptr) return fail(APK_ERR_ARG, "null buffer");
  if (((reinterpret_cast<uintptr_t>(shard) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) return fail(APK_ERR_ARG, "buffers must be 16-byte aligned");
  apk::CParams cp;
  int rc = coll_common(comm, shard_bytes, shard_bytes, &cp, stream);
  if (rc != APK_OK) return rc;
  cp.src = reinterpret_cast<const uint8_t*>(shard);
  cp.out = reinterpret_cast<uint8_t*>(out);
  cp.flag_stride = apk::FLAG_STRIDE;
  for (int r = 0; r < comm->world && comm->world > 1; ++r) cp.flag_peer[r] = reinterpret_cast<uint32_t*>(comm->flags[r]);
  cp.flag_local = comm->world > 1 ? cp.flag_peer[comm->rank] : nullptr;
  return launch_collective(apk::all_gather_kernel, cp, stream);
}

int apk_reduce_scatter(const apk_comm* comm, const void* in, void* out, uint64_t out_bytes, int32_t dtype, int32_t reduce_op, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (out_bytes == 0) return APK_OK;
  if (in == nullptr || out == nullptr) return fail(APK_ERR_ARG, "null buffer");
  if (dtype != APK_BF16 && dtype != APK_F32) return fail(APK_ERR_ARG, "dtype must be bf16 or f32");
  if (reduce_op != APK_REDUCE_SUM && reduce_op != APK_REDUCE_AVG) return fail(APK_ERR_ARG, "reduce_op must be sum or avg");
  if (((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) != 0) return fail(APK_ERR_ARG, "buffers must be 16-byte aligned");
  if (comm == nullptr) return fail(APK_ERR_ARG, "comm is null");
  apk::CParams cp;
  int rc = coll_common(comm, out_bytes, out_bytes * (uint64_t)comm->world, &cp, stream);
  if (rc != APK_OK) return rc;
  cp.src = reinterpret_cast<const uint8_t*>(in);
  cp.out = reinterpret_cast<uint8_t*>(out);
  cp.fp32 = dtype == APK_F32;
  cp.reduce_scale = reduce_op == APK_REDUCE_AVG ? 1.0f / (float)comm->world : 1.0f;
  if (comm->world > 1) {
    const uint64_t max_tiles = (comm->flag_bytes - kFlagRsOffset) / 4 / (uint64_t)comm->world;
    cp.flag_stride = (int32_t)max_tiles;   // flag (source, tile 0) of the per-tile flag array
    for (int r = 0; r < comm->world; ++r) cp.flag_peer[r] = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(comm->flags[r]) + kFlagRsOffset);
    cp.flag_local = cp.flag_peer[comm->rank];
  }
  return launch_collective(apk::reduce_scatter_kernel, cp, stream);
}

static int g_debug_rs_lag = 0;
void apk_debug_set_rs_lag(int32_t row_blocks) { g_debug_rs_lag = row_blocks; }

int apk_debug_schedule(int32_t mode, int32_t world, int32_t rank, int32_t rows_per_rank, int32_t nB, const int32_t* N,
                       int32_t last_dim, int32_t pair, int32_t crank, int32_t* out, int32_t capacity) {
  if (nB < 1 || nB > APK_MAX_B || N == nullptr || world < 1 || world > APK_MAX_WORLD) return fail(APK_ERR_ARG, "bad arguments");
  apk::KParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.mode = mode;
  kp.ws = world;
  kp.rank = rank;
  kp.nB = nB;
  kp.rows_per_rank = rows_per_rank;
  kp.ag_ksplit = (mode == apk::MODE_AG && last_dim) ? 1 : 0;
  kp.rs_colsplit = (mode == apk::MODE_RS && last_dim) ? 1 : 0;
  kp.rs_lag = g_debug_rs_lag;
  int max_n = 0;
  for (int b = 0; b < nB; ++b) {
    kp.N[b] = N[b];
    max_n = N[b] > max_n ? N[b] : max_n;
  }
  if (max_n <= 128) return pair ? fail(APK_ERR_ARG, "pairs need 256-column tiles") : schedule_rows<128, false>(kp, 0, out, capacity);
  return pair ? schedule_rows<256, true>(kp, crank, out, capacity) : schedule_rows<256, false>(kp, 0, out, capacity);
}

int apk_check_status(const apk_comm* comm, void* stream_, uint32_t* raw) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (comm == nullptr || comm->status == nullptr) return fail(APK_ERR_ARG, "comm.status is null");
  uint32_t v = 0;
  APK_CUDA(cudaMemcpyAsync(&v, comm->status, 4, cudaMemcpyDeviceToHost, stream));
  APK_CUDA(cudaStreamSynchronize(stream));
  if (raw != nullptr) *raw = v;
  if (v != 0) {
    APK_CUDA(cudaMemsetAsync(comm->status, 0, 4, stream));
    APK_CUDA(cudaStreamSynchronize(stream));
    static const char* names[] = {"ok", "pipeline mbarrier", "peer 'staged' flag", "gathered rows", "peer partial"};
    const uint32_t code = v & 0xffu;
    return fail(APK_ERR_TIMEOUT, "device wait timed out: %s (detail %u)", code < 5 ? names[code] : "?", v >> 8);
  }
  return APK_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// apk_ag_gemm_static: the same all-gather matmul, with the library's own fixed scratch.
//
// Scratch that apk_ag_gemm expects from its caller (the per-call counters behind comm->ctrl, the
// gathered copy of A when the caller does not want it back, the gathered row scales) lives here
// in one file-scope device array instead. The array exists once per GPU that loads the library
// and is shared by every call on that GPU.
// ---------------------------------------------------------------------------------------------
namespace {

constexpr uint64_t kStaticCtrlBytes = 64ull << 10;       // per-call counters
constexpr uint64_t kStaticScaleBytes = 256ull << 10;     // gathered row scales: up to 65536 rows
constexpr uint64_t kStaticGatheredBytes = 32ull << 20;   // gathered A: world * rows_per_rank * K * element size
constexpr uint64_t kStaticTotal = kStaticCtrlBytes + kStaticScaleBytes + kStaticGatheredBytes;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticTotal];

// Device address of g_static_scratch on the current device. In host code the array's name is
// only a handle for the runtime, so the address is asked for once per device.
int static_scratch_base(unsigned char** out) {
  static unsigned char* base[64] = {};
  static std::mutex mu;
  int dev = 0;
  APK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(APK_ERR_ARG, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (base[dev] == nullptr) {
    void* p = nullptr;
    APK_CUDA(cudaGetSymbolAddress(&p, g_static_scratch));
    if (p == nullptr) return fail(APK_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
    base[dev] = static_cast<unsigned char*>(p);
  }
  *out = base[dev];
  return APK_OK;
}

}  // namespace

extern "C" int apk_ag_gemm_static(const apk_comm* comm, const apk_ag_gemm_args* a, void* stream_) {
  if (comm == nullptr) return fail(APK_ERR_ARG, "comm is null");
  if (a == nullptr) return fail(APK_ERR_ARG, "args is null");
  if (a->rows_per_rank < 0 || a->K <= 0 || comm->world < 1 || comm->world > APK_MAX_WORLD)
    return fail(APK_ERR_ARG, "bad shape or group size");
  const uint64_t es = a->dtype == APK_E4M3 ? 1 : 2;
  const uint64_t rows = (uint64_t)a->rows_per_rank * (uint64_t)comm->world;
  const uint64_t gathered = rows * (uint64_t)a->K * es;
  const uint64_t ctrl = apk_ctrl_bytes(a->rows_per_rank, comm->world);
  if (!a->return_A && comm->world > 1 && gathered > kStaticGatheredBytes)
    return fail(APK_ERR_SIZE, "apk_ag_gemm_static: the gathered A needs %llu bytes, the fixed scratch holds %llu; use apk_ag_gemm",
                (unsigned long long)gathered, (unsigned long long)kStaticGatheredBytes);
  if (a->a_scale_mode == APK_SCALE_VECTOR && rows * 4 > kStaticScaleBytes)
    return fail(APK_ERR_SIZE, "apk_ag_gemm_static: %llu gathered rows, the fixed scratch holds scales for %llu; use apk_ag_gemm",
                (unsigned long long)rows, (unsigned long long)(kStaticScaleBytes / 4));
  if (ctrl > kStaticCtrlBytes)
    return fail(APK_ERR_SIZE, "apk_ag_gemm_static: %llu bytes of counters needed, the fixed scratch holds %llu; use apk_ag_gemm",
                (unsigned long long)ctrl, (unsigned long long)kStaticCtrlBytes);
  unsigned char* base = nullptr;
  int rc = static_scratch_base(&base);
  if (rc != APK_OK) return rc;
  apk_comm c = *comm;
  c.ctrl = base;                      // zeroed by apk_ag_gemm for the part each call uses
  c.ctrl_bytes = kStaticCtrlBytes;
  apk_ag_gemm_args args = *a;
  args.A_scale_gathered = reinterpret_cast<float*>(base + kStaticCtrlBytes);
  if (!a->return_A) args.A_gathered = base + kStaticCtrlBytes + kStaticScaleBytes;
  return apk_ag_gemm(&c, &args, stream_);
}
