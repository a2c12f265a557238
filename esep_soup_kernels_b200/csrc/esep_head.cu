// C ABI of libesep_head.so: argument checks, work decomposition, TMA descriptors and launches.
// The entry points are declared and documented in include/esep_head.h.

#include "../../include/esep_head.h"

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstring>
#include <mutex>

#include "head_aux.cuh"
#include "head_bwd.cuh"
#include "head_dx.cuh"
#include "head_fwd.cuh"
#include "head_norm.cuh"
#include "head_step.cuh"
#include "head_train.cuh"
#include "head_train_wide.cuh"
#include "head_weight.cuh"

using namespace esep;

namespace {

constexpr int kMaxDevices = 64;
constexpr int kBwdCluster = 4;
constexpr size_t kAlign = 256;

struct DeviceInfo {
  int cc_major = 0, cc_minor = 0, sm_count = 0, max_clusters_bwd = 0, max_pairs_fwd = 0;
  int max_clusters_wide = 0;   // resident 8-CTA clusters of head_train_wide_kernel (0: not available)
  int max_pairs_dx = 0;        // resident CTA pairs of head_dx_kernel (0: not available)
  int init_status = ESEP_ERR_CUDA;
};

// Per-device init-once table. `g_ready` is set only when the initialisation reached a final
// verdict (ok, or a device that can never run the kernels); a transient CUDA failure leaves it
// clear, so the next call tries again instead of failing for the life of the process.
std::mutex g_init_mutex;
std::atomic<int> g_ready[kMaxDevices];
DeviceInfo g_info[kMaxDevices];
PFN_cuTensorMapEncodeTiled g_encode = nullptr;
std::atomic<long long> g_init_calls{0};   // completed per-device initialisations (test aid)
std::atomic<long long> g_launches{0};     // kernels this library has launched (all entry points)
std::atomic<long long> g_wide_launches{0};   // of head_train_wide_kernel
std::atomic<long long> g_dx_launches{0};     // of head_dx_kernel
std::atomic<int> g_training_path{0};          // esep_head_set_training_path
constexpr size_t kMaxStoredLogitsBytes = static_cast<size_t>(48) << 30;

size_t align_up(size_t x) { return (x + kAlign - 1) / kAlign * kAlign; }

// Set by esep_head_train around its guarded second attempt: every kernel the forward / finalize /
// backward entry points launch meanwhile carries this device flag and does nothing when it is 0.
thread_local const int* g_gate = nullptr;

void load_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) ==
          cudaSuccess &&
      qres == cudaDriverEntryPointSuccess)
    g_encode = reinterpret_cast<PFN_cuTensorMapEncodeTiled>(fn);
}

template <typename K>
cudaError_t set_smem(K kernel, int bytes) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// Runs under g_init_mutex. Returns true when the verdict in g_info[device] is final.
bool init_device(int device) {
  DeviceInfo d;
  int prev = -1;
  if (cudaGetDevice(&prev) != cudaSuccess) return false;
  if (cudaSetDevice(device) != cudaSuccess) return false;
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
    cudaSetDevice(prev);
    return false;
  }
  d.cc_major = prop.major;
  d.cc_minor = prop.minor;
  d.sm_count = prop.multiProcessorCount;
  if (prop.major != 10) {
    d.init_status = ESEP_ERR_UNSUPPORTED_ARCH;
    g_info[device] = d;
    cudaSetDevice(prev);
    return true;
  }
  if (g_encode == nullptr) load_encode();
  bool ok = g_encode != nullptr;
  ok = ok && set_smem(head_fwd_kernel<0>, fwd::SMEM_BYTES) == cudaSuccess;
  ok = ok && set_smem(head_fwd_kernel<1>, fwd::SMEM_BYTES) == cudaSuccess;
  ok = ok && set_smem(head_bwd_kernel<0>, bwd::SMEM_BYTES) == cudaSuccess;
  ok = ok && set_smem(head_bwd_kernel<1>, bwd::SMEM_BYTES) == cudaSuccess;
  ok = ok && set_smem(head_train_kernel<0>, trn::SMEM_BYTES_T) == cudaSuccess;
  ok = ok && set_smem(head_train_kernel<1>, trn::SMEM_BYTES_T) == cudaSuccess;
  if (ok) {
    // How many CTA pairs of the forward kernel can be resident at once.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(d.sm_count / 2 * 2));
    cfg.blockDim = dim3(fwd::THREADS);
    cfg.dynamicSmemBytes = fwd::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int npairs = 0;
    if (cudaOccupancyMaxActiveClusters(&npairs, head_fwd_kernel<0>, &cfg) == cudaSuccess &&
        npairs > 0)
      d.max_pairs_fwd = std::min(npairs, d.sm_count / 2);
    else
      ok = false;
  }
  if (ok) {
    // How many 4-CTA clusters of the backward kernel can be resident at once.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(d.sm_count / kBwdCluster * kBwdCluster));
    cfg.blockDim = dim3(bwd::THREADS);
    cfg.dynamicSmemBytes = bwd::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = kBwdCluster;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int ncl = 0;
    if (cudaOccupancyMaxActiveClusters(&ncl, head_bwd_kernel<0>, &cfg) ==
            cudaSuccess &&
        ncl > 0)
      d.max_clusters_bwd = std::min(ncl, d.sm_count / kBwdCluster);
    else
      ok = false;
  }
  if (ok) {
    // How many 8-CTA clusters of the wide training kernel can be resident at once. A device that
    // cannot place one keeps the 4-CTA kernel for every hidden size: not an error.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(d.sm_count / trnw::CLW * trnw::CLW));
    cfg.blockDim = dim3(trn::THREADS_T);
    cfg.dynamicSmemBytes = trn::SMEM_BYTES_T;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = trnw::CLW;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int ncl = 0;
    if (cudaFuncSetAttribute(head_train_wide_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             trn::SMEM_BYTES_T) == cudaSuccess &&
        cudaFuncSetAttribute(head_train_wide_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             trn::SMEM_BYTES_T) == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&ncl, head_train_wide_kernel<0>, &cfg) == cudaSuccess &&
        ncl > 0)
      d.max_clusters_wide = std::min(ncl, d.sm_count / trnw::CLW);
  }
  if (ok) {
    // CTA pairs of the dHidden-from-stored-logits kernel, and the attributes of the storing sweep.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(d.sm_count / 2 * 2));
    cfg.blockDim = dim3(dxk::THREADS);
    cfg.dynamicSmemBytes = dxk::SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int npairs = 0;
    if (cudaFuncSetAttribute(head_dx_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             dxk::SMEM_BYTES) == cudaSuccess &&
        cudaFuncSetAttribute(head_dx_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             dxk::SMEM_BYTES) == cudaSuccess &&
        cudaFuncSetAttribute(head_dx_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             dxk::SMEM_BYTES) == cudaSuccess &&
        cudaFuncSetAttribute(head_fwd_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fwd::SMEM_BYTES) == cudaSuccess &&
        cudaFuncSetAttribute(head_fwd_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fwd::SMEM_BYTES) == cudaSuccess &&
        cudaFuncSetAttribute(head_fwd_kernel<0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fwd::SMEM_BYTES_STORE) == cudaSuccess &&
        cudaFuncSetAttribute(head_fwd_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             fwd::SMEM_BYTES_STORE) == cudaSuccess &&
        cudaOccupancyMaxActiveClusters(&npairs, head_dx_kernel<0>, &cfg) == cudaSuccess &&
        npairs > 0)
      d.max_pairs_dx = std::min(npairs, d.sm_count / 2);
  }
  cudaGetLastError();
  cudaSetDevice(prev);
  if (!ok) return false;
  d.init_status = ESEP_OK;
  g_info[device] = d;
  return true;
}

int device_info(int device, const DeviceInfo** out) {
  if (device < 0 || device >= kMaxDevices) return ESEP_ERR_BAD_ARG;
  if (g_ready[device].load(std::memory_order_acquire) == 0) {
    std::lock_guard<std::mutex> lock(g_init_mutex);
    if (g_ready[device].load(std::memory_order_relaxed) == 0) {
      if (!init_device(device)) {
        cudaGetLastError();
        *out = nullptr;
        return ESEP_ERR_CUDA;   // nothing is remembered: the next call tries again
      }
      g_init_calls.fetch_add(1);
      g_ready[device].store(1, std::memory_order_release);
    }
  }
  *out = &g_info[device];
  return g_info[device].init_status;
}

int current_device_info(const DeviceInfo** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return ESEP_ERR_CUDA;
  }
  return device_info(dev, out);
}

// Encoded tensor maps are kept in a small table keyed on everything that goes into them (the
// counterpart of the reference's per-weight cache, solution/head/patch.py:93-101: the head weight
// and the library's own buffers keep their addresses from step to step). A map is address
// arithmetic only, so an entry can never go stale: the same key always encodes the same map.
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols;
  uint32_t box[3];
  int dtype, dims;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box[0] == o.box[0] &&
           box[1] == o.box[1] && box[2] == o.box[2] && dtype == o.dtype && dims == o.dims;
  }
};
constexpr int kTmapSlots = 64;
std::mutex g_tmap_mutex;
TmapKey g_tmap_keys[kTmapSlots];
CUtensorMap g_tmap_vals[kTmapSlots];
int g_tmap_used = 0, g_tmap_next = 0;
std::atomic<long long> g_tmap_encodes{0};

bool tmap_lookup(const TmapKey& key, CUtensorMap* map) {
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  for (int i = 0; i < g_tmap_used; ++i)
    if (g_tmap_keys[i] == key) {
      *map = g_tmap_vals[i];
      return true;
    }
  return false;
}
void tmap_store(const TmapKey& key, const CUtensorMap& map) {
  std::lock_guard<std::mutex> lock(g_tmap_mutex);
  const int slot = g_tmap_used < kTmapSlots ? g_tmap_used++ : (g_tmap_next++ % kTmapSlots);
  g_tmap_keys[slot] = key;
  g_tmap_vals[slot] = map;
}

int make_tmap_uncached(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows, uint64_t cols,
                       uint32_t box_cols, uint32_t box_rows);
int make_tmap_w3_uncached(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows,
                          uint64_t cols, uint32_t box_rows, uint32_t box_blocks);

// 2-D row-major 16-bit tensor [rows, cols], box {box_cols, box_rows}, 128-byte swizzle,
// out-of-bounds elements read as zero.
int make_tmap(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows, uint64_t cols,
              uint32_t box_cols, uint32_t box_rows) {
  const TmapKey key = {ptr, rows, cols, {box_cols, box_rows, 0}, dtype, 2};
  if (tmap_lookup(key, map)) return ESEP_OK;
  const int st = make_tmap_uncached(map, ptr, dtype, rows, cols, box_cols, box_rows);
  if (st == ESEP_OK) tmap_store(key, *map);
  return st;
}

int make_tmap_uncached(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows, uint64_t cols,
                       uint32_t box_cols, uint32_t box_rows) {
  g_tmap_encodes.fetch_add(1);
  const cuuint64_t gdim[2] = {cols, rows};
  const cuuint64_t gstride[1] = {cols * 2};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt =
      dtype == ESEP_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = g_encode(map, dt, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ESEP_OK : ESEP_ERR_CUDA;
}

// W [v, h] viewed as {64 h, v, h / 64} (h % 64 == 0): one box {64, box_rows, box_blocks} lands in
// shared memory as box_blocks consecutive 64-wide tiles of box_rows lines.
int make_tmap_w3(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows, uint64_t cols,
                 uint32_t box_rows, uint32_t box_blocks) {
  const TmapKey key = {ptr, rows, cols, {64, box_rows, box_blocks}, dtype, 3};
  if (tmap_lookup(key, map)) return ESEP_OK;
  const int st = make_tmap_w3_uncached(map, ptr, dtype, rows, cols, box_rows, box_blocks);
  if (st == ESEP_OK) tmap_store(key, *map);
  return st;
}

int make_tmap_w3_uncached(CUtensorMap* map, const void* ptr, int dtype, uint64_t rows,
                          uint64_t cols, uint32_t box_rows, uint32_t box_blocks) {
  g_tmap_encodes.fetch_add(1);
  const cuuint64_t gdim[3] = {64, rows, cols / 64};
  const cuuint64_t gstride[2] = {cols * 2, 128};
  const cuuint32_t box[3] = {64, box_rows, box_blocks};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUtensorMapDataType dt =
      dtype == ESEP_DTYPE_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = g_encode(map, dt, 3, const_cast<void*>(ptr), gdim, gstride, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? ESEP_OK : ESEP_ERR_CUDA;
}

int check_problem(const void* x, const void* w, int64_t n, int64_t h, int64_t v, int dtype) {
  if (x == nullptr || w == nullptr) return ESEP_ERR_BAD_ARG;
  if (n <= 0 || h <= 0 || v <= 0) return ESEP_ERR_BAD_ARG;
  if (n > (1 << 30) || v > (1 << 30) || h > (1 << 20)) return ESEP_ERR_BAD_ARG;
  if (h % 8 != 0) return ESEP_ERR_BAD_ARG;
  if (dtype != ESEP_DTYPE_F16 && dtype != ESEP_DTYPE_BF16) return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(w) & 15u))
    return ESEP_ERR_ALIGNMENT;
  return ESEP_OK;
}

int div_up(int64_t a, int64_t b) { return static_cast<int>((a + b - 1) / b); }

}  // namespace

extern "C" {

const char* esep_head_status_string(int code) {
  switch (code) {
    case ESEP_OK: return "ok";
    case ESEP_ERR_BAD_ARG: return "bad argument (null pointer, shape, dtype, or h % 8 != 0)";
    case ESEP_ERR_UNSUPPORTED_ARCH: return "device is not compute capability 10.x (sm_100a)";
    case ESEP_ERR_WORKSPACE: return "workspace null, misaligned or too small";
    case ESEP_ERR_CUDA: return "CUDA runtime/driver call failed";
    case ESEP_ERR_DEVICE_TIMEOUT: return "a kernel gave up on a bounded wait";
    case ESEP_ERR_ALIGNMENT: return "x or W is not 16-byte aligned";
    case ESEP_ERR_STATIC_SCRATCH:
      return "problem needs more scratch than the built-in static array holds";
    default: return "unknown status";
  }
}

int esep_head_query(int device, esep_head_caps* caps) {
  if (caps == nullptr) return ESEP_ERR_BAD_ARG;
  const DeviceInfo* d = nullptr;
  const int st = device_info(device, &d);
  if (d == nullptr) {
    caps->cc_major = caps->cc_minor = caps->sm_count = caps->max_clusters_bwd = 0;
    caps->supported = 0;
    return st;
  }
  caps->cc_major = d->cc_major;
  caps->cc_minor = d->cc_minor;
  caps->sm_count = d->sm_count;
  caps->max_clusters_bwd = d->max_clusters_bwd;
  caps->supported = (st == ESEP_OK) ? 1 : 0;
  return st;
}

int esep_head_warmup(int device) {
  const DeviceInfo* d = nullptr;
  return device_info(device, &d);
}

int esep_head_plan_problem(int64_t n, int64_t h, int64_t v_local, int need_grad, int sm_count,
                           int max_clusters_bwd, esep_head_plan* plan) {
  if (plan == nullptr || n <= 0 || h <= 0 || v_local <= 0 || sm_count <= 0)
    return ESEP_ERR_BAD_ARG;
  if (n > (1 << 30) || v_local > (1 << 30) || h > (1 << 20) || h % 8 != 0) return ESEP_ERR_BAD_ARG;
  esep_head_plan pl = {};
  // ---- forward: units = row-tile pairs x runs of vocabulary tiles, persistent CTA pairs ----
  pl.fwd_row_tiles = div_up(n, fwd::BM);
  pl.fwd_vocab_tiles = div_up(v_local, fwd::BN);
  {
    const int row_pairs = div_up(pl.fwd_row_tiles, 2);
    const int pairs = std::max(1, sm_count / 2);
    const double ideal = static_cast<double>(row_pairs) * pl.fwd_vocab_tiles / pairs;
    int best_tpu = 1;
    double best_eff = -1.0;
    for (int tpu = pl.fwd_vocab_tiles; tpu >= 1; --tpu) {
      const int splits = div_up(pl.fwd_vocab_tiles, tpu);
      if (splits > 2048) break;
      const int64_t units = static_cast<int64_t>(row_pairs) * splits;
      const double t = static_cast<double>((units + pairs - 1) / pairs) * tpu;
      const double eff = ideal / t;
      if (eff > best_eff + 1e-9) {
        best_eff = eff;
        best_tpu = tpu;
      }
      if (eff >= 0.97) break;  // prefer the coarsest split that balances the SMs
    }
    pl.fwd_tiles_per_unit = best_tpu;
    pl.fwd_splits = div_up(pl.fwd_vocab_tiles, best_tpu);
    const int64_t units = static_cast<int64_t>(row_pairs) * pl.fwd_splits;
    pl.fwd_grid = 2 * static_cast<int>(std::min<int64_t>(units, pairs));
  }
  // ---- backward: clusters of 4 CTAs (two CTA pairs), each CTA one H-slice -----------------
  pl.bwd_cluster = kBwdCluster;
  {
    int nhb = div_up(h, kBwdCluster * 128);
    if (nhb > 3) nhb = 3;
    pl.bwd_hblocks = nhb;
    pl.bwd_hslice = nhb * 128;
    pl.bwd_passes = div_up(h, static_cast<int64_t>(kBwdCluster) * pl.bwd_hslice);
    pl.bwd_total_steps = div_up(v_local, bwd::STEP_V);
    // Full rounds (every cluster sweeps one whole (row tile, pass)) plus one balanced last
    // round: each of the left-over pairs is cut into as many vocabulary runs as there are
    // clusters per left-over pair, one run per cluster, and comes out as partial pieces.
    const int64_t n_tp = static_cast<int64_t>(pl.fwd_row_tiles) * pl.bwd_passes;
    const int ncl = static_cast<int>(std::min<int64_t>(
        std::max(1, max_clusters_bwd), n_tp * pl.bwd_total_steps));
    pl.bwd_grid = ncl * kBwdCluster;
    const SweepSplit sp = sweep_split(n_tp, ncl, pl.bwd_total_steps);
    pl.bwd_full_rounds = sp.full_rounds;
    pl.bwd_rem_pairs = sp.rem_tp;
    pl.bwd_rem_splits = sp.rem_splits;
    pl.bwd_steps_per_split = sp.steps_per_split;
  }
  // ---- workspace -------------------------------------------------------------------------
  size_t off = 0;
  pl.ws_status_off = off;
  off += kAlign;
  pl.ws_partial_off = off;
  off += align_up(static_cast<size_t>(5) * pl.fwd_splits * n * sizeof(float));
  pl.ws_record_off = off;
  off += align_up(static_cast<size_t>(ESEP_RECORD_FIELDS) * n * sizeof(float));
  pl.ws_cew_off = off;
  off += align_up(static_cast<size_t>(n) * sizeof(float));
  pl.ws_dxpart_off = off;
  if (need_grad && pl.bwd_rem_pairs > 0)
    off += align_up(static_cast<size_t>(pl.bwd_rem_splits) * pl.bwd_rem_pairs * 128 *
                    kBwdCluster * pl.bwd_hslice * sizeof(float));
  pl.ws_bytes = off;
  *plan = pl;
  return ESEP_OK;
}

size_t esep_head_workspace_bytes(int64_t n, int64_t h, int64_t v_local, int dtype, int need_grad) {
  (void)dtype;
  const DeviceInfo* d = nullptr;
  if (current_device_info(&d) != ESEP_OK) return 0;
  esep_head_plan pl;
  if (esep_head_plan_problem(n, h, v_local, need_grad, d->sm_count, d->max_clusters_bwd, &pl) !=
      ESEP_OK)
    return 0;
  return pl.ws_bytes;
}

int esep_head_forward_partial(const void* x, const void* w, const int64_t* target, int64_t n,
                              int64_t h, int64_t v_local, int64_t vocab_offset, int dtype,
                              float* record, void* workspace, size_t workspace_bytes,
                              void* stream) {
  int st = check_problem(x, w, n, h, v_local, dtype);
  if (st != ESEP_OK) return st;
  if (target == nullptr || record == nullptr) return ESEP_ERR_BAD_ARG;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  esep_head_plan pl;
  st = esep_head_plan_problem(n, h, v_local, 0, d->sm_count, d->max_clusters_bwd, &pl);
  if (st != ESEP_OK) return st;
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) ||
      workspace_bytes < pl.ws_bytes)
    return ESEP_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  int* status = reinterpret_cast<int*>(ws + pl.ws_status_off);
  if (g_gate == nullptr && cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess)
    return ESEP_ERR_CUDA;

  CUtensorMap tx, tw;
  if (make_tmap(&tx, x, dtype, n, h, fwd::BK, fwd::BM) != ESEP_OK) return ESEP_ERR_CUDA;
  if (make_tmap(&tw, w, dtype, v_local, h, fwd::BK, fwd::BN / 2) != ESEP_OK) return ESEP_ERR_CUDA;

  FwdParams p;
  p.n = static_cast<int>(n);
  p.h = static_cast<int>(h);
  p.v = static_cast<int>(v_local);
  p.n_row_tiles = pl.fwd_row_tiles;
  p.n_row_pairs = div_up(pl.fwd_row_tiles, 2);
  p.n_vtiles = pl.fwd_vocab_tiles;
  p.tiles_per_unit = pl.fwd_tiles_per_unit;
  p.n_splits = pl.fwd_splits;
  p.vocab_offset = vocab_offset;
  p.target = reinterpret_cast<const long long*>(target);
  float* part = reinterpret_cast<float*>(ws + pl.ws_partial_off);
  const size_t pn = static_cast<size_t>(pl.fwd_splits) * n;
  p.pm = part;
  p.ps = part + pn;
  p.pt = part + 2 * pn;
  p.ptz = part + 3 * pn;
  p.pidx = reinterpret_cast<int*>(part + 4 * pn);
  p.status = status;
  p.gate = g_gate;
  p.row_range = nullptr;
  p.part_cap = 0;

  {
    // The kernel strides its work units by the number of launched pairs, so clamping the grid
    // to what can be resident at once only changes the balance, never the result.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(std::min(pl.fwd_grid, 2 * d->max_pairs_fwd)));
    cfg.blockDim = dim3(fwd::THREADS);
    cfg.dynamicSmemBytes = fwd::SMEM_BYTES;
    cfg.stream = s;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const cudaError_t e = dtype == ESEP_DTYPE_F16
                              ? cudaLaunchKernelEx(&cfg, head_fwd_kernel<0>, tx, tw, tw, p)
                              : cudaLaunchKernelEx(&cfg, head_fwd_kernel<1>, tx, tw, tw, p);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return ESEP_ERR_CUDA;
    }
    g_launches.fetch_add(1);
  }

  const int threads = 256;
  head_merge_kernel<<<div_up(n, threads), threads, 0, s>>>(p.n, pl.fwd_splits, p.pm, p.ps, p.pt,
                                                           p.ptz, p.pidx, vocab_offset, record,
                                                           g_gate);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_finalize(const float* records, int n_records, const int64_t* target,
                       const float* ce_weight, int64_t n, int64_t v_global, float* lse,
                       float* target_logit, float* ce, float* entropy, int64_t* argmax,
                       float* cew_out, float* loss, float* metrics, void* workspace,
                       size_t workspace_bytes, void* stream) {
  if (records == nullptr || target == nullptr || ce_weight == nullptr || lse == nullptr ||
      target_logit == nullptr || ce == nullptr || entropy == nullptr || argmax == nullptr ||
      cew_out == nullptr || loss == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (n <= 0 || n > (1 << 30) || v_global <= 0 || n_records <= 0) return ESEP_ERR_BAD_ARG;
  const int* status = nullptr;
  if (workspace != nullptr) {
    if ((reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) || workspace_bytes < kAlign)
      return ESEP_ERR_WORKSPACE;
    status = reinterpret_cast<const int*>(workspace);
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  head_rows_kernel<<<div_up(n, threads), threads, 0, s>>>(
      static_cast<int>(n), n_records, v_global, records,
      reinterpret_cast<const long long*>(target), ce_weight, lse, target_logit, ce, entropy,
      reinterpret_cast<long long*>(argmax), cew_out, g_gate);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  head_scalars_kernel<<<1, 1024, 0, s>>>(static_cast<int>(n), v_global, ce, cew_out, entropy,
                                         reinterpret_cast<const long long*>(argmax),
                                         reinterpret_cast<const long long*>(target), status, loss,
                                         metrics, g_gate);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_forward(const void* x, const void* w, const int64_t* target, const float* ce_weight,
                      int64_t n, int64_t h, int64_t v, int dtype, float* lse, float* target_logit,
                      float* ce, float* entropy, int64_t* argmax, float* cew_out, float* loss,
                      float* metrics, void* workspace, size_t workspace_bytes, void* stream) {
  int st = check_problem(x, w, n, h, v, dtype);
  if (st != ESEP_OK) return st;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  esep_head_plan pl;
  st = esep_head_plan_problem(n, h, v, 0, d->sm_count, d->max_clusters_bwd, &pl);
  if (st != ESEP_OK) return st;
  if (workspace == nullptr || workspace_bytes < pl.ws_bytes) return ESEP_ERR_WORKSPACE;
  float* record = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + pl.ws_record_off);
  st = esep_head_forward_partial(x, w, target, n, h, v, 0, dtype, record, workspace,
                                 workspace_bytes, stream);
  if (st != ESEP_OK) return st;
  return esep_head_finalize(record, 1, target, ce_weight, n, v, lse, target_logit, ce, entropy,
                            argmax, cew_out, loss, metrics, workspace, workspace_bytes, stream);
}

int esep_head_backward(const void* x, const void* w, const int64_t* target, const float* cew,
                       const float* lse, int64_t n, int64_t h, int64_t v_local,
                       int64_t vocab_offset, int dtype, float* dx, void* workspace,
                       size_t workspace_bytes, void* stream) {
  int st = check_problem(x, w, n, h, v_local, dtype);
  if (st != ESEP_OK) return st;
  if (target == nullptr || cew == nullptr || lse == nullptr || dx == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(dx) & 15u) return ESEP_ERR_ALIGNMENT;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  esep_head_plan pl;
  st = esep_head_plan_problem(n, h, v_local, 1, d->sm_count, d->max_clusters_bwd, &pl);
  if (st != ESEP_OK) return st;
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) ||
      workspace_bytes < pl.ws_bytes)
    return ESEP_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* ws = static_cast<uint8_t*>(workspace);

  CUtensorMap tx, tw1, tw2;
  if (make_tmap(&tx, x, dtype, n, h, bwd::BK, 64) != ESEP_OK) return ESEP_ERR_CUDA;
  if (make_tmap(&tw1, w, dtype, v_local, h, bwd::BK, bwd::BV) != ESEP_OK) return ESEP_ERR_CUDA;
  const bool w2_is_3d = (h % 64 == 0);
  if (w2_is_3d) {
    if (make_tmap_w3(&tw2, w, dtype, v_local, h, bwd::G2_KV, 6) != ESEP_OK) return ESEP_ERR_CUDA;
  } else if (make_tmap(&tw2, w, dtype, v_local, h, 64, bwd::G2_KV) != ESEP_OK) {
    return ESEP_ERR_CUDA;
  }

  BwdParams p;
  p.n = static_cast<int>(n);
  p.h = static_cast<int>(h);
  p.v = static_cast<int>(v_local);
  p.n_row_tiles = pl.fwd_row_tiles;
  p.nhb = pl.bwd_hblocks;
  p.n_passes = pl.bwd_passes;
  p.total_steps = pl.bwd_total_steps;
  p.full_rounds = pl.bwd_full_rounds;
  p.rem_tp = pl.bwd_rem_pairs;
  p.rem_splits = pl.bwd_rem_splits;
  p.steps_per_split = pl.bwd_steps_per_split;
  p.dx_part = reinterpret_cast<float*>(ws + pl.ws_dxpart_off);
  p.vocab_offset = vocab_offset;
  p.target = reinterpret_cast<const long long*>(target);
  p.cew = cew;
  p.lse = lse;
  p.w = w;
  p.dx = dx;
  p.p_scale = dtype == ESEP_DTYPE_F16 ? 1024.f : 1.f;
  p.w2_is_3d = w2_is_3d ? 1 : 0;
  p.status = reinterpret_cast<int*>(ws + pl.ws_status_off);
  p.gate = g_gate;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(pl.bwd_grid));
  cfg.blockDim = dim3(bwd::THREADS);
  cfg.dynamicSmemBytes = bwd::SMEM_BYTES;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = kBwdCluster;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  cudaError_t e;
  if (dtype == ESEP_DTYPE_F16)
    e = cudaLaunchKernelEx(&cfg, head_bwd_kernel<0>, tx, tw1, tw2, p);
  else
    e = cudaLaunchKernelEx(&cfg, head_bwd_kernel<1>, tx, tw1, tw2, p);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return ESEP_ERR_CUDA;
  }
  g_launches.fetch_add(1);
  if (pl.bwd_rem_pairs > 0) {
    head_dx_sum_kernel<<<pl.bwd_rem_pairs * 128, 128, 0, s>>>(
        p.n, p.h, pl.fwd_row_tiles, pl.bwd_full_rounds * (pl.bwd_grid / kBwdCluster),
        pl.bwd_rem_pairs, pl.bwd_rem_splits, kBwdCluster * pl.bwd_hslice, p.dx_part, dx, g_gate);
    if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  }
  return ESEP_OK;
}

int esep_head_selftest_bounded_wait(void* workspace, size_t workspace_bytes, int64_t limit_cycles,
                                    void* stream) {
  if (workspace == nullptr || (reinterpret_cast<uintptr_t>(workspace) & (kAlign - 1)) ||
      workspace_bytes < kAlign)
    return ESEP_ERR_WORKSPACE;
  if (limit_cycles <= 0 || limit_cycles > 2000000000LL) return ESEP_ERR_BAD_ARG;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int* status = static_cast<int*>(workspace);
  if (cudaMemsetAsync(status, 0, sizeof(int), s) != cudaSuccess) return ESEP_ERR_CUDA;
  head_wait_probe_kernel<<<1, 32, 0, s>>>(status, limit_cycles);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_device_status(const void* workspace, void* stream, int* out_status) {
  if (workspace == nullptr || out_status == nullptr) return ESEP_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  if (cudaMemcpyAsync(&v, workspace, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return ESEP_ERR_CUDA;
  }
  *out_status = v;
  return v == 0 ? ESEP_OK : ESEP_ERR_DEVICE_TIMEOUT;
}


// ---------------------------------------------------------------------------------------------
// Forward without a caller-provided workspace: the scratch lives in a fixed array that is part
// of the loaded module. See esep_head_forward_static in include/esep_head.h.
// ---------------------------------------------------------------------------------------------
}  // extern "C"

namespace {
// Per-GPU scratch of the static entry point. Every device that loads the library carries these
// 16 MiB until the process exits. In host code the symbol below is only a handle; its device
// address is looked up once per device with cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_static_scratch[ESEP_STATIC_SCRATCH_BYTES];
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the scratch array on `device`, which must be current. Looked up once per
// device; a failed lookup is not remembered, so a later call can try again. No allocation.
void* resolve_static_scratch(int device) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[device] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) == cudaSuccess) g_static_ptr[device] = ptr;
    else cudaGetLastError();
  }
  return g_static_ptr[device];
}
}  // namespace

extern "C" {

size_t esep_head_static_scratch_bytes(void) { return ESEP_STATIC_SCRATCH_BYTES; }

int esep_head_forward_static(const void* x, const void* w, const int64_t* target,
                             const float* ce_weight, int64_t n, int64_t h, int64_t v, int dtype,
                             float* lse, float* target_logit, float* ce, float* entropy,
                             int64_t* argmax, float* cew_out, float* loss, float* metrics,
                             void* stream) {
  int st = check_problem(x, w, n, h, v, dtype);
  if (st != ESEP_OK) return st;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  esep_head_plan pl;
  st = esep_head_plan_problem(n, h, v, 0, d->sm_count, d->max_clusters_bwd, &pl);
  if (st != ESEP_OK) return st;
  if (pl.ws_bytes > ESEP_STATIC_SCRATCH_BYTES) return ESEP_ERR_STATIC_SCRATCH;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ESEP_ERR_CUDA;
  void* scratch = resolve_static_scratch(dev);
  if (scratch == nullptr) return ESEP_ERR_CUDA;
  // The forward clears the status word itself; every other scratch cell it reads is written
  // earlier in the same call, so nothing else has to start at zero.
  return esep_head_forward(x, w, target, ce_weight, n, h, v, dtype, lse, target_logit, ce, entropy,
                           argmax, cew_out, loss, metrics, scratch, ESEP_STATIC_SCRATCH_BYTES,
                           stream);
}

}  // extern "C"



// ---------------------------------------------------------------------------------------------
// The final residual add + RMSNorm in front of the head and its backward (head_norm.cuh).
// ---------------------------------------------------------------------------------------------
// Block size and float4s per thread for a row of `nvec` float4s: every thread gets work.
#define ESEP_NORM_SHAPE(nvec, LAUNCH)          \
  if ((nvec) <= 128) { LAUNCH(128, 1) }        \
  else if ((nvec) <= 256) { LAUNCH(128, 2) }   \
  else if ((nvec) <= 384) { LAUNCH(128, 3) }   \
  else if ((nvec) <= 512) { LAUNCH(128, 4) }   \
  else if ((nvec) <= 768) { LAUNCH(256, 3) }   \
  else if ((nvec) <= 1024) { LAUNCH(256, 4) }  \
  else if ((nvec) <= 1536) { LAUNCH(256, 6) }  \
  else { LAUNCH(256, 8) }

namespace {
int check_norm(int64_t n, int64_t h, int dtype, std::initializer_list<const void*> required,
               std::initializer_list<const void*> aligned) {
  if (n < 0 || h <= 0 || n > (1 << 30)) return ESEP_ERR_BAD_ARG;
  if (h % 4 != 0 || h > esep::norm::MAX_H) return ESEP_ERR_BAD_ARG;
  if (dtype != ESEP_DTYPE_F16 && dtype != ESEP_DTYPE_BF16) return ESEP_ERR_BAD_ARG;
  if (n == 0) return ESEP_OK;
  for (const void* q : required)
    if (q == nullptr) return ESEP_ERR_BAD_ARG;
  for (const void* q : aligned)
    if (reinterpret_cast<uintptr_t>(q) & 15u) return ESEP_ERR_ALIGNMENT;
  return ESEP_OK;
}
}  // namespace

extern "C" {

int esep_head_norm_forward(const float* r_in, const void* delta, const float* gamma, int64_t n,
                           int64_t h, float eps, int dtype, float* r_out, void* y, float* rstd,
                           void* stream) {
  int st = check_norm(n, h, dtype, {r_in, gamma, y, rstd}, {r_in, delta, gamma, r_out, y});
  if (st != ESEP_OK) return st;
  if (delta != nullptr && r_out == nullptr) return ESEP_ERR_BAD_ARG;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  if (n == 0) return ESEP_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(n));
  const int hi = static_cast<int>(h);
  const int variant = (dtype == ESEP_DTYPE_F16 ? 0 : 2) + (delta != nullptr ? 1 : 0);
#define ESEP_NORM_FWD(F, D, T, M) \
  esep::head_norm_fwd_kernel<F, D, T, M><<<grid, T, 0, s>>>(r_in, delta, gamma, hi, eps, r_out, y, rstd)
#define ESEP_NORM_FWD_V(T, M)                         \
  switch (variant) {                                  \
    case 0: ESEP_NORM_FWD(0, false, T, M); break;     \
    case 1: ESEP_NORM_FWD(0, true, T, M); break;      \
    case 2: ESEP_NORM_FWD(1, false, T, M); break;     \
    default: ESEP_NORM_FWD(1, true, T, M); break;     \
  }
  ESEP_NORM_SHAPE(h / 4, ESEP_NORM_FWD_V)
#undef ESEP_NORM_FWD_V
#undef ESEP_NORM_FWD
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_norm_backward(const float* dy, const float* r_out, const float* rstd,
                            const float* gamma, const float* dr_out, int64_t n, int64_t h,
                            int dtype, float* dr, void* ddelta, void* stream) {
  int st = check_norm(n, h, dtype, {dy, r_out, rstd, gamma, dr}, {dy, r_out, gamma, dr_out, dr, ddelta});
  if (st != ESEP_OK) return st;
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  if (n == 0) return ESEP_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(static_cast<unsigned>(n));
  const int hi = static_cast<int>(h);
  const int variant = (dtype == ESEP_DTYPE_F16 ? 0 : 4) + (dr_out != nullptr ? 2 : 0) +
                      (ddelta != nullptr ? 1 : 0);
#define ESEP_NORM_BWD(F, A, B, T, M)                                                        \
  esep::head_norm_bwd_kernel<F, A, B, T, M><<<grid, T, 0, s>>>(dy, r_out, rstd, gamma, dr_out, hi, \
                                                                dr, ddelta)
#define ESEP_NORM_BWD_V(T, M)                               \
  switch (variant) {                                        \
    case 0: ESEP_NORM_BWD(0, false, false, T, M); break;    \
    case 1: ESEP_NORM_BWD(0, false, true, T, M); break;     \
    case 2: ESEP_NORM_BWD(0, true, false, T, M); break;     \
    case 3: ESEP_NORM_BWD(0, true, true, T, M); break;      \
    case 4: ESEP_NORM_BWD(1, false, false, T, M); break;    \
    case 5: ESEP_NORM_BWD(1, false, true, T, M); break;     \
    case 6: ESEP_NORM_BWD(1, true, false, T, M); break;     \
    default: ESEP_NORM_BWD(1, true, true, T, M); break;     \
  }
  ESEP_NORM_SHAPE(h / 4, ESEP_NORM_BWD_V)
#undef ESEP_NORM_BWD_V
#undef ESEP_NORM_BWD
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

}  // extern "C"




// ---------------------------------------------------------------------------------------------
// Whole head step: row classes decided on the device, one pass over the vocabulary for the rows
// that need a gradient (head_train.cuh), a forward sweep for the rest, outputs in the caller's
// row order (head_step.cuh). Workspace = the regular plan's workspace (used by the host-planned
// prefix sweep and by the guarded two-kernel pass) followed by the step's own arrays.
// ---------------------------------------------------------------------------------------------
namespace {
constexpr int64_t kPrefixRows = 2048;   // vocabulary prefix that gives the per-row reference maximum

struct StepLayout {
  esep_head_plan pl;   // host plan for all m rows with gradient
  int ncl;             // clusters of the training sweep launch
  bool wide;           // the sweep runs as 8-CTA clusters (head_train_wide_kernel), one pass
  int nhb_a, nhb_b;    // wide: accumulator blocks per producer / consumer CTA
  int rows_nhb;        // accumulator blocks per quarter of a pass, as the row-finish kernel sees it
  int pass_w;          // columns per pass = row stride of the partial dHidden pieces
  bool stored;         // two sweeps: forward sweep that keeps a 16-bit value per logit, then head_dx_kernel
  bool direct;         // ... stores the softmax weights themselves (bf16), head_dx_kernel<.., true>
  size_t zpitch;       // elements per row of that buffer
  size_t z_off, c2_off, partg_off, pieces_off;
  int part_cap;        // rows of the forward partial arrays
  size_t base_bytes;
  size_t record_off, st_off, st_stride, lo_off, lo_stride, dxpart_off, xc_off, tgtc_off, tgto_off,
      cewc_off, perm_off, inv_off, dxc_off, part_off, part_stride, fb_off, fb_stride, fbam_off,
      floss_off, total;
};

int step_layout(int64_t m, int64_t h, int64_t v, bool need_grad, const DeviceInfo* d,
                StepLayout* t) {
  int st = esep_head_plan_problem(m, h, v, 1, d->sm_count, d->max_clusters_bwd, &t->pl);
  if (st != ESEP_OK) return st;
  esep_head_plan pre;
  st = esep_head_plan_problem(m, h, std::min<int64_t>(v, kPrefixRows), 0, d->sm_count,
                              d->max_clusters_bwd, &pre);
  if (st != ESEP_OK) return st;
  const esep_head_plan& pl = t->pl;
  t->ncl = pl.bwd_grid / kBwdCluster;
  t->wide = false;
  t->nhb_a = t->nhb_b = 0;
  t->rows_nhb = pl.bwd_hblocks;
  t->pass_w = kBwdCluster * pl.bwd_hslice;
  // Hidden sizes of three passes whose accumulator fits eight SMs (28 blocks of 128 columns). With
  // two passes the 4-CTA kernel is the faster one (measured: 645 - 670 against 561 - 614 TFLOP/s
  // algorithmic at 2048 - 3072 columns; at 3584: 456 against 621).
  if (need_grad && d->max_clusters_wide > 0 && pl.bwd_passes > 2 && h % 128 == 0 &&
      h <= 28 * 128) {
    const int blocks = static_cast<int>(h / 128);
    t->wide = true;
    t->nhb_a = div_up(std::max(blocks - 16, 1), 4);
    t->nhb_b = div_up(blocks - 4 * t->nhb_a, 4);
    t->rows_nhb = div_up(blocks, 4);
    t->pass_w = 4 * t->rows_nhb * 128;
    const int64_t n_tp = div_up(m, 128);
    t->ncl = static_cast<int>(
        std::min<int64_t>(d->max_clusters_wide, n_tp * pl.bwd_total_steps));
  }
  t->stored = t->direct = false;
  t->zpitch = static_cast<size_t>(pl.fwd_vocab_tiles) * 256;
  {
    const int path = g_training_path.load();
    const size_t zbytes = static_cast<size_t>(m) * t->zpitch * 2;
    // Measured on B200 (same box, alternating), 4 340 x 1536 x 151 936: single pass 3.55 ms, two
    // sweeps over fp16 logits 3.39 ms, two sweeps over bf16 softmax weights 2.91 ms; 7B shard shape
    // (32 768 x 3584 x 19 008): 13.5 / 8.9 - 9.4 / 7.7 - 8.7 ms. The two sweeps are the default
    // wherever they apply; the single pass remains for callers that cannot spare the buffer.
    if (need_grad && path != 1 && d->max_pairs_dx > 0 && h % 64 == 0 &&
        zbytes <= kMaxStoredLogitsBytes)
      t->stored = true;
    t->direct = t->stored && path != 2;   // path 2: fp16 logits, transformed by the dHidden kernel
  }
  const size_t mr = static_cast<size_t>(div_up(m, 256)) * 256;
  // Rows of the forward partial arrays: room for 16 vocabulary runs per row (the split search of
  // fwd_split_rows then reaches 97 % of the pairs for any row count: with 3 runs, 128 row pairs on
  // 74 CTA pairs lose 13 % to the last wave), bounded for very large batches.
  {
    const size_t few = mr + static_cast<size_t>(4) * 256 * d->max_pairs_fwd;
    const size_t many = std::min<size_t>(16 * mr, static_cast<size_t>(1) << 22);
    t->part_cap = static_cast<int>(std::min<size_t>(std::max(few, many), static_cast<size_t>(1) << 30));
  }
  const size_t f4 = sizeof(float);
  size_t off = align_up(std::max(pl.ws_bytes, pre.ws_bytes));
  t->base_bytes = off;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align_up(bytes);
    return at;
  };
  t->tgto_off = take(static_cast<size_t>(m) * 8);
  t->tgtc_off = take(static_cast<size_t>(m) * 8);
  t->cewc_off = take(static_cast<size_t>(m) * f4);
  t->perm_off = take(static_cast<size_t>(m) * 4);
  t->inv_off = take(static_cast<size_t>(m) * 4);
  t->xc_off = take(static_cast<size_t>(m) * h * 2);
  t->part_stride = align_up(static_cast<size_t>(t->part_cap) * f4);
  t->part_off = take(5 * t->part_stride);
  // what only a call with gradient needs
  t->record_off = off;
  t->st_off = t->lo_off = t->dxpart_off = t->dxc_off = t->fb_off = t->fbam_off = t->floss_off = off;
  t->st_stride = t->lo_stride = t->fb_stride = 0;
  if (need_grad) t->record_off = take(static_cast<size_t>(ESEP_RECORD_FIELDS) * m * f4);
  if (need_grad && !t->stored) {
    t->st_stride = align_up(static_cast<size_t>(16) * m * f4);
    t->st_off = take(4 * t->st_stride);
    // a left-over pair is cut into at most ncl / rem_tp runs: rem_tp * rem_splits <= ncl
    t->lo_stride = align_up(static_cast<size_t>(16) * 128 * t->ncl * f4);
    t->lo_off = take(4 * t->lo_stride);
    t->dxpart_off = take(static_cast<size_t>(t->ncl) * 128 * t->pass_w * f4);
  }
  if (need_grad && (!t->stored || t->direct)) {   // what the guarded second attempt leaves
    t->dxc_off = take(static_cast<size_t>(m) * h * f4);
    t->fb_stride = align_up(static_cast<size_t>(m) * f4);
    t->fb_off = take(5 * t->fb_stride);
    t->fbam_off = take(static_cast<size_t>(m) * 8);
    t->floss_off = take(kAlign);
  }
  t->z_off = t->c2_off = t->partg_off = t->pieces_off = off;
  if (t->stored) {
    t->z_off = take(static_cast<size_t>(m) * t->zpitch * 2);
    t->c2_off = take(2 * align_up(static_cast<size_t>(m) * f4));   // kexp, rscale
    t->partg_off = take(5 * t->part_stride);
    t->pieces_off = take(static_cast<size_t>(dx_max_runs(static_cast<int>(m), static_cast<int>(h),
                                                         static_cast<int>(v), d->max_pairs_dx)) *
                         dxk::ROWS * dxk::SLICE * f4);
  }
  t->total = off;
  return ESEP_OK;
}

struct StepArgs {
  const void* x;
  int x_dtype;               // ESEP_DTYPE_F16 / BF16 (= dtype) or ESEP_DTYPE_F32
  const void* w;
  const void* w_bf16;        // bf16 copy of W for the dHidden GEMM (w itself for bf16 models)
  int dtype;
  int64_t m, h, v;
  const int64_t* target;     // flat rows
  const float* ce_weight;
  const int64_t* labels;     // or a [batch, seq_len] step
  const int64_t* attention_mask;
  int64_t seq_len;
  int need_grad;
  float *lse, *target_logit, *ce, *entropy, *cew_out, *loss, *metrics, *dx, *top_logit;
  int64_t* argmax;
  int* overflow;             // may be null
  void* workspace;
  size_t workspace_bytes;
  void* stream;
};

template <typename K, typename... A>
int launch_cluster(K kernel, unsigned grid, unsigned block, size_t smem, unsigned cluster,
                   cudaStream_t s, A... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = cluster;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kernel, args...) != cudaSuccess) {
    cudaGetLastError();
    return ESEP_ERR_CUDA;
  }
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int step_impl(const StepArgs& a) {
  int st = check_problem(a.x, a.w, a.m, a.h, a.v, a.dtype);
  if (st != ESEP_OK) return st;
  const bool step_mode = a.labels != nullptr;
  if (!step_mode && a.target == nullptr) return ESEP_ERR_BAD_ARG;
  if (step_mode && (a.seq_len <= 0 || a.m % a.seq_len != 0)) return ESEP_ERR_BAD_ARG;
  if (a.x_dtype != a.dtype && a.x_dtype != ESEP_DTYPE_F32) return ESEP_ERR_BAD_ARG;
  if (a.lse == nullptr || a.target_logit == nullptr || a.ce == nullptr || a.entropy == nullptr ||
      a.argmax == nullptr || a.cew_out == nullptr || a.loss == nullptr)
    return ESEP_ERR_BAD_ARG;
  const bool need_grad = a.need_grad != 0;
  if (need_grad) {
    if (a.dx == nullptr) return ESEP_ERR_BAD_ARG;
    if ((reinterpret_cast<uintptr_t>(a.dx) & 15u) || (reinterpret_cast<uintptr_t>(a.w_bf16) & 15u))
      return ESEP_ERR_ALIGNMENT;
  }
  const DeviceInfo* d = nullptr;
  st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  StepLayout t;
  st = step_layout(a.m, a.h, a.v, need_grad, d, &t);
  if (st != ESEP_OK) return st;
  // the bf16 copy of W is read by the single pass only (the two sweeps read W in its own type)
  if (need_grad && (!t.stored || (t.direct && a.dtype == ESEP_DTYPE_F16)) && a.w_bf16 == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (a.workspace == nullptr || (reinterpret_cast<uintptr_t>(a.workspace) & (kAlign - 1)) ||
      a.workspace_bytes < t.total)
    return ESEP_ERR_WORKSPACE;
  cudaStream_t s = static_cast<cudaStream_t>(a.stream);
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  const esep_head_plan& pl = t.pl;
  const int m = static_cast<int>(a.m), h = static_cast<int>(a.h), v = static_cast<int>(a.v);
  int* status = reinterpret_cast<int*>(ws + pl.ws_status_off);
  int* counts = reinterpret_cast<int*>(ws + 64);          // inside the status block
  int* overflow = a.overflow != nullptr ? a.overflow : reinterpret_cast<int*>(ws + 96);
  long long* tgt_o = reinterpret_cast<long long*>(ws + t.tgto_off);
  long long* tgt_c = reinterpret_cast<long long*>(ws + t.tgtc_off);
  float* cew_c = reinterpret_cast<float*>(ws + t.cewc_off);
  int* perm = reinterpret_cast<int*>(ws + t.perm_off);
  int* inv = reinterpret_cast<int*>(ws + t.inv_off);
  void* xc = ws + t.xc_off;
  float* part = reinterpret_cast<float*>(ws + t.part_off);
  float* record = reinterpret_cast<float*>(ws + t.record_off);
  float* dxc = reinterpret_cast<float*>(ws + t.dxc_off);

  // 1. row classes, compact order, counts (device only)
  StepPrepParams q = {};
  q.m = m;
  q.v = v;
  q.seq_len = static_cast<int>(step_mode ? a.seq_len : 1);
  q.need_grad = need_grad ? 1 : 0;
  q.target = reinterpret_cast<const long long*>(a.target);
  q.ce_weight = a.ce_weight;
  q.labels = reinterpret_cast<const long long*>(a.labels);
  q.attn = reinterpret_cast<const long long*>(a.attention_mask);
  q.tgt_o = tgt_o;
  q.tgt_c = tgt_c;
  q.cew_c = cew_c;
  q.perm = perm;
  q.inv = inv;
  q.counts = counts;
  q.overflow = overflow;
  q.status = status;
  q.stored = t.stored ? 1 : 0;
  head_step_prep_kernel<<<1, 1024, 0, s>>>(q);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);

  // 2. compact 16-bit copy of the selected rows
  {
    const bool f32 = a.x_dtype == ESEP_DTYPE_F32;
    const unsigned grid = static_cast<unsigned>(m);
    if (a.dtype == ESEP_DTYPE_F16) {
      if (f32) head_step_gather_kernel<0, true><<<grid, 128, 0, s>>>(a.x, perm, h, xc);
      else head_step_gather_kernel<0, false><<<grid, 128, 0, s>>>(a.x, perm, h, xc);
    } else {
      if (f32) head_step_gather_kernel<1, true><<<grid, 128, 0, s>>>(a.x, perm, h, xc);
      else head_step_gather_kernel<1, false><<<grid, 128, 0, s>>>(a.x, perm, h, xc);
    }
    if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  }

  const size_t st_stride = t.st_stride, lo_stride = t.lo_stride;
  TrainParams p = {};
  if (need_grad) {
    // 3. reference maximum per row: the forward sweep over a vocabulary prefix (record field 0).
    //    Host-planned over all m compact rows; the rows past n_sel hold zeros.
    g_gate = nullptr;
    st = esep_head_forward_partial(xc, a.w, reinterpret_cast<const int64_t*>(tgt_c), a.m, a.h,
                                   std::min<int64_t>(a.v, kPrefixRows), 0, a.dtype, record,
                                   a.workspace, t.base_bytes, a.stream);
    if (st != ESEP_OK) return st;

  }
  const unsigned fwd_grid = static_cast<unsigned>(2 * d->max_pairs_fwd);
  float* part_g = reinterpret_cast<float*>(ws + t.partg_off);
  const size_t psg = t.part_stride / sizeof(float);
  if (need_grad && t.stored) {
    // 4a. forward sweep over the compact rows [0, n_sweep) that keeps the softmax weights as bf16
    //     (direct) or logit - m_ref as fp16
    CUtensorMap tx, tw;
    if (make_tmap(&tx, xc, a.dtype, a.m, a.h, fwd::BK, fwd::BM) != ESEP_OK) return ESEP_ERR_CUDA;
    if (make_tmap(&tw, a.w, a.dtype, a.v, a.h, fwd::BK, fwd::BN / 2) != ESEP_OK)
      return ESEP_ERR_CUDA;
    FwdParams g = {};
    g.n = m;
    g.h = h;
    g.v = v;
    g.n_row_tiles = pl.fwd_row_tiles;
    g.n_row_pairs = div_up(pl.fwd_row_tiles, 2);
    g.n_vtiles = pl.fwd_vocab_tiles;
    g.tiles_per_unit = pl.fwd_tiles_per_unit;
    g.n_splits = pl.fwd_splits;
    g.vocab_offset = 0;
    g.target = tgt_c;
    g.pm = part_g;
    g.ps = part_g + psg;
    g.pt = part_g + 2 * psg;
    g.ptz = part_g + 3 * psg;
    g.pidx = reinterpret_cast<int*>(part_g + 4 * psg);
    g.status = status;
    g.gate = nullptr;
    g.row_range = counts + CNT_ZERO;   // {0, n_sweep}
    g.part_cap = t.part_cap;
    g.zbuf = reinterpret_cast<__half*>(ws + t.z_off);
    g.zpitch = static_cast<long long>(t.zpitch);
    g.m_ref = record;
    if (t.direct) {
      CUtensorMap tzs;   // the weights buffer as the epilogue warps store it: boxes of 64 x 32 rows
      if (make_tmap(&tzs, g.zbuf, ESEP_DTYPE_BF16, a.m, t.zpitch, 64, 32) != ESEP_OK)
        return ESEP_ERR_CUDA;
      st = a.dtype == ESEP_DTYPE_F16
               ? launch_cluster(head_fwd_kernel<0, 2>, fwd_grid, fwd::THREADS,
                                fwd::SMEM_BYTES_STORE, 2, s, tx, tw, tzs, g)
               : launch_cluster(head_fwd_kernel<1, 2>, fwd_grid, fwd::THREADS,
                                fwd::SMEM_BYTES_STORE, 2, s, tx, tw, tzs, g);
    } else {
      st = a.dtype == ESEP_DTYPE_F16
               ? launch_cluster(head_fwd_kernel<0, 1>, fwd_grid, fwd::THREADS, fwd::SMEM_BYTES, 2,
                                s, tx, tw, tw, g)
               : launch_cluster(head_fwd_kernel<1, 1>, fwd_grid, fwd::THREADS, fwd::SMEM_BYTES, 2,
                                s, tx, tw, tw, g);
    }
    if (st != ESEP_OK) return st;
    // 4b. per-row constant of the softmax weights, 4c. dHidden from the stored buffer
    float* kexp = reinterpret_cast<float*>(ws + t.c2_off);
    float* rscale = reinterpret_cast<float*>(ws + t.c2_off + align_up(static_cast<size_t>(m) * sizeof(float)));
    const unsigned rc_grid = static_cast<unsigned>(div_up(m, 128));
    head_dx_rowconst_kernel<<<rc_grid, 128, 0, s>>>(m, counts + CNT_STORE, pl.fwd_vocab_tiles,
                                                    static_cast<int>(fwd_grid / 2), t.part_cap, g.pm,
                                                    g.ps, g.ptz, tgt_c, v, record, kexp, rscale,
                                                    t.direct ? 1 : 0, overflow);
    if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
    g_launches.fetch_add(1);
    CUtensorMap tw3, tz;
    if (t.direct) {   // P is bf16: an fp16 model's dHidden GEMM reads the bf16 copy of W
      const void* wb = a.dtype == ESEP_DTYPE_F16 ? a.w_bf16 : a.w;
      if (make_tmap_w3(&tw3, wb, ESEP_DTYPE_BF16, a.v, a.h, dxk::KV, 4) != ESEP_OK)
        return ESEP_ERR_CUDA;
      if (make_tmap(&tz, g.zbuf, ESEP_DTYPE_BF16, a.m, t.zpitch, 64, 128) != ESEP_OK)
        return ESEP_ERR_CUDA;
    } else {
      if (make_tmap_w3(&tw3, a.w, a.dtype, a.v, a.h, dxk::KV, 4) != ESEP_OK) return ESEP_ERR_CUDA;
      tz = tw3;
    }
    DxParams dp = {};
    dp.n = m;
    dp.h = h;
    dp.v = v;
    dp.n_dev = counts + CNT_STORE;
    dp.z = g.zbuf;
    dp.zpitch = g.zpitch;
    dp.kexp = kexp;
    dp.target = tgt_c;
    dp.pieces = reinterpret_cast<float*>(ws + t.pieces_off);
    dp.status = status;
    const unsigned dx_grid = static_cast<unsigned>(2 * d->max_pairs_dx);
    if (t.direct)
      st = launch_cluster(head_dx_kernel<1, true>, dx_grid, dxk::THREADS, dxk::SMEM_BYTES, 2, s,
                          tw3, tz, dp);
    else
      st = a.dtype == ESEP_DTYPE_F16
               ? launch_cluster(head_dx_kernel<0>, dx_grid, dxk::THREADS, dxk::SMEM_BYTES, 2, s,
                                tw3, tz, dp)
               : launch_cluster(head_dx_kernel<1>, dx_grid, dxk::THREADS, dxk::SMEM_BYTES, 2, s,
                                tw3, tz, dp);
    if (st != ESEP_OK) return st;
    g_dx_launches.fetch_add(1);
  }
  if (need_grad && !t.stored) {
    // 4. the training sweep over the compact rows [0, n_sweep)
    CUtensorMap tx, tw1, tw2, tw2b;
    if (make_tmap(&tx, xc, a.dtype, a.m, a.h, bwd::BK, 64) != ESEP_OK) return ESEP_ERR_CUDA;
    if (make_tmap(&tw1, a.w, a.dtype, a.v, a.h, bwd::BK, bwd::BV) != ESEP_OK) return ESEP_ERR_CUDA;
    const bool w2_is_3d = (a.h % 64 == 0);
    if (w2_is_3d) {
      if (make_tmap_w3(&tw2, a.w_bf16, ESEP_DTYPE_BF16, a.v, a.h, bwd::G2_KV, 6) != ESEP_OK)
        return ESEP_ERR_CUDA;
    } else if (make_tmap(&tw2, a.w_bf16, ESEP_DTYPE_BF16, a.v, a.h, 64, bwd::G2_KV) != ESEP_OK) {
      return ESEP_ERR_CUDA;
    }
    p.n = m;
    p.h = h;
    p.v = v;
    p.n_dev = counts + CNT_TRAIN;
    p.nhb = pl.bwd_hblocks;
    p.total_steps = pl.bwd_total_steps;
    p.m_ref = record;
    p.target = tgt_c;
    p.dx = dxc;
    p.dx_part = reinterpret_cast<float*>(ws + t.dxpart_off);
    p.st_s = reinterpret_cast<float*>(ws + t.st_off);
    p.st_t = reinterpret_cast<float*>(ws + t.st_off + st_stride);
    p.st_max = reinterpret_cast<float*>(ws + t.st_off + 2 * st_stride);
    p.st_idx = reinterpret_cast<int*>(ws + t.st_off + 3 * st_stride);
    p.lo_s = reinterpret_cast<float*>(ws + t.lo_off);
    p.lo_t = reinterpret_cast<float*>(ws + t.lo_off + lo_stride);
    p.lo_max = reinterpret_cast<float*>(ws + t.lo_off + 2 * lo_stride);
    p.lo_idx = reinterpret_cast<int*>(ws + t.lo_off + 3 * lo_stride);
    p.w2_is_3d = w2_is_3d ? 1 : 0;
    p.overflow = overflow;
    p.status = status;
    if (t.wide) {
      // one pass on 8-CTA clusters: same arrays, same work split, other geometry
      if (make_tmap_w3(&tw2, a.w_bf16, ESEP_DTYPE_BF16, a.v, a.h, bwd::G2_KV, 2 * t.nhb_a) !=
              ESEP_OK ||
          make_tmap_w3(&tw2b, a.w_bf16, ESEP_DTYPE_BF16, a.v, a.h, bwd::G2_KV, 2 * t.nhb_b) !=
              ESEP_OK)
        return ESEP_ERR_CUDA;
      TrainWideParams pw = {};
      pw.n = m;
      pw.h = h;
      pw.v = v;
      pw.n_dev = p.n_dev;
      pw.nhb_a = t.nhb_a;
      pw.nhb_b = t.nhb_b;
      pw.pass_w = t.pass_w;
      pw.slots_a = 4;   // measured at 3584 columns: 2 / 3 / 4 / 5 slots -> 389 / 562 / 640 / 612 TFLOP/s
      pw.total_steps = p.total_steps;
      pw.m_ref = p.m_ref;
      pw.target = p.target;
      pw.dx = p.dx;
      pw.dx_part = p.dx_part;
      pw.st_s = p.st_s; pw.st_t = p.st_t; pw.st_max = p.st_max; pw.st_idx = p.st_idx;
      pw.lo_s = p.lo_s; pw.lo_t = p.lo_t; pw.lo_max = p.lo_max; pw.lo_idx = p.lo_idx;
      pw.overflow = overflow;
      pw.status = status;
      const unsigned grid = static_cast<unsigned>(t.ncl * trnw::CLW);
      st = a.dtype == ESEP_DTYPE_F16
               ? launch_cluster(head_train_wide_kernel<0>, grid, trn::THREADS_T, trn::SMEM_BYTES_T,
                                trnw::CLW, s, tx, tw1, tw2, tw2b, pw)
               : launch_cluster(head_train_wide_kernel<1>, grid, trn::THREADS_T, trn::SMEM_BYTES_T,
                                trnw::CLW, s, tx, tw1, tw2, tw2b, pw);
      if (st == ESEP_OK) g_wide_launches.fetch_add(1);
    } else {
      st = a.dtype == ESEP_DTYPE_F16
               ? launch_cluster(head_train_kernel<0>, static_cast<unsigned>(pl.bwd_grid),
                                trn::THREADS_T, trn::SMEM_BYTES_T, kBwdCluster, s, tx, tw1, tw2, p)
               : launch_cluster(head_train_kernel<1>, static_cast<unsigned>(pl.bwd_grid),
                                trn::THREADS_T, trn::SMEM_BYTES_T, kBwdCluster, s, tx, tw1, tw2, p);
    }
    if (st != ESEP_OK) return st;
  }

  // 5. forward sweep over the compact rows [n_sweep, n_sel): statistics only
  FwdParams f = {};
  {
    CUtensorMap tx, tw;
    if (make_tmap(&tx, xc, a.dtype, a.m, a.h, fwd::BK, fwd::BM) != ESEP_OK) return ESEP_ERR_CUDA;
    if (make_tmap(&tw, a.w, a.dtype, a.v, a.h, fwd::BK, fwd::BN / 2) != ESEP_OK)
      return ESEP_ERR_CUDA;
    f.n = m;
    f.h = h;
    f.v = v;
    f.n_row_tiles = pl.fwd_row_tiles;
    f.n_row_pairs = div_up(pl.fwd_row_tiles, 2);
    f.n_vtiles = pl.fwd_vocab_tiles;
    f.tiles_per_unit = pl.fwd_tiles_per_unit;
    f.n_splits = pl.fwd_splits;
    f.vocab_offset = 0;
    f.target = tgt_c;
    const size_t ps = t.part_stride / sizeof(float);
    f.pm = part;
    f.ps = part + ps;
    f.pt = part + 2 * ps;
    f.ptz = part + 3 * ps;
    f.pidx = reinterpret_cast<int*>(part + 4 * ps);
    f.status = status;
    f.gate = nullptr;
    f.row_range = counts + CNT_SWEEP;   // {n_sweep, n_sel}
    f.part_cap = t.part_cap;
    st = a.dtype == ESEP_DTYPE_F16
             ? launch_cluster(head_fwd_kernel<0>, fwd_grid, fwd::THREADS, fwd::SMEM_BYTES, 2, s, tx,
                              tw, tw, f)
             : launch_cluster(head_fwd_kernel<1>, fwd_grid, fwd::THREADS, fwd::SMEM_BYTES, 2, s, tx,
                              tw, tw, f);
    if (st != ESEP_OK) return st;
  }

  float* fb = reinterpret_cast<float*>(ws + t.fb_off);
  const size_t fbs = t.fb_stride / sizeof(float);
  long long* fb_amax = reinterpret_cast<long long*>(ws + t.fbam_off);
  if (need_grad && (!t.stored || t.direct)) {
    // 6. guarded second attempt on the compact rows: the two-kernel path, enqueued behind the
    //    overflow flag. Its kernels return at once unless a row overflowed in the sweep; if one
    //    did, they leave per-row results and final dHidden rows in compact order.
    g_gate = overflow;
    st = esep_head_forward(xc, a.w, reinterpret_cast<const int64_t*>(tgt_c), cew_c, a.m, a.h, a.v,
                           a.dtype, fb, fb + fbs, fb + 2 * fbs, fb + 3 * fbs,
                           reinterpret_cast<int64_t*>(fb_amax), fb + 4 * fbs,
                           reinterpret_cast<float*>(ws + t.floss_off), nullptr, a.workspace,
                           t.base_bytes, a.stream);
    if (st == ESEP_OK)
      st = esep_head_backward(xc, a.w, reinterpret_cast<const int64_t*>(tgt_c), fb + 4 * fbs, fb,
                              a.m, a.h, a.v, 0, a.dtype, dxc, a.workspace, t.base_bytes, a.stream);
    g_gate = nullptr;
    if (st != ESEP_OK) return st;
  }

  // 7. per-row finish in the caller's row order, 8. the scalars
  StepRowsParams r = {};
  r.m = m;
  r.h = h;
  r.v = v;
  r.n_clusters = t.ncl;
  r.nhb = t.rows_nhb;
  r.total_steps = pl.bwd_total_steps;
  r.n_vtiles = pl.fwd_vocab_tiles;
  r.fwd_pairs = static_cast<int>(fwd_grid / 2);
  r.part_cap = t.part_cap;
  r.counts = counts;
  r.overflow = overflow;
  r.inv = inv;
  r.xc = xc;
  r.w = a.w;
  r.tgt_c = tgt_c;
  r.cew_c = cew_c;
  r.m_ref = record;
  r.st_s = p.st_s; r.st_t = p.st_t; r.st_max = p.st_max; r.st_idx = p.st_idx;
  r.lo_s = p.lo_s; r.lo_t = p.lo_t; r.lo_max = p.lo_max; r.lo_idx = p.lo_idx;
  r.dx_part = p.dx_part;
  r.dxc = dxc;
  r.pm = f.pm; r.ps = f.ps; r.pt = f.pt; r.ptz = f.ptz; r.pidx = f.pidx;
  r.f_lse = fb; r.f_tl = fb + fbs; r.f_ce = fb + 2 * fbs; r.f_ent = fb + 3 * fbs;
  r.f_cew = fb + 4 * fbs;
  r.f_max = reinterpret_cast<const float*>(ws + pl.ws_record_off);   // esep_head_forward's record
  r.f_amax = fb_amax;
  r.lse = a.lse; r.tlogit = a.target_logit; r.ce = a.ce; r.ent = a.entropy; r.cew_out = a.cew_out;
  r.amax = reinterpret_cast<long long*>(a.argmax);
  r.top = a.top_logit;
  r.dx = need_grad ? a.dx : nullptr;
  r.stored = (need_grad && t.stored) ? 1 : 0;
  r.dx_pairs = d->max_pairs_dx;
  r.g_rscale = reinterpret_cast<const float*>(ws + t.c2_off + align_up(static_cast<size_t>(a.m) * sizeof(float)));
  r.g_pm = part_g;
  r.g_ps = part_g + psg;
  r.g_pt = part_g + 2 * psg;
  r.g_ptz = part_g + 3 * psg;
  r.g_pidx = reinterpret_cast<const int*>(part_g + 4 * psg);
  r.pieces = reinterpret_cast<const float*>(ws + t.pieces_off);
  if (a.dtype == ESEP_DTYPE_F16)
    head_step_rows_kernel<0><<<static_cast<unsigned>(m), 128, 0, s>>>(r);
  else
    head_step_rows_kernel<1><<<static_cast<unsigned>(m), 128, 0, s>>>(r);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  head_step_scalars_kernel<<<1, 1024, 0, s>>>(m, a.v, a.ce, a.cew_out, a.entropy,
                                              reinterpret_cast<const long long*>(a.argmax), tgt_o,
                                              step_mode ? q.attn : nullptr, counts, status, a.loss,
                                              a.metrics);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}
}  // namespace

extern "C" {

size_t esep_head_step_workspace_bytes(int64_t m, int64_t h, int64_t v, int dtype, int need_grad) {
  if (m <= 0 || h <= 0 || v <= 0 || h % 8 != 0) return 0;
  if (dtype != ESEP_DTYPE_F16 && dtype != ESEP_DTYPE_BF16) return 0;
  const DeviceInfo* d = nullptr;
  if (current_device_info(&d) != ESEP_OK) return 0;
  StepLayout t;
  if (step_layout(m, h, v, need_grad != 0, d, &t) != ESEP_OK) return 0;
  return t.total;
}

int esep_head_step(const void* x, int x_dtype, const void* w, const void* w_bf16, int dtype,
                   int64_t m, int64_t h, int64_t v, const int64_t* target, const float* ce_weight,
                   const int64_t* labels, const int64_t* attention_mask, int64_t seq_len,
                   int need_grad, float* lse, float* target_logit, float* ce, float* entropy,
                   int64_t* argmax, float* cew_out, float* loss, float* metrics, float* dx,
                   float* top_logit, int* overflow, void* workspace, size_t workspace_bytes,
                   void* stream) {
  StepArgs a = {};
  a.x = x; a.x_dtype = x_dtype; a.w = w; a.w_bf16 = w_bf16; a.dtype = dtype;
  a.m = m; a.h = h; a.v = v;
  a.target = target; a.ce_weight = ce_weight; a.labels = labels;
  a.attention_mask = attention_mask; a.seq_len = seq_len; a.need_grad = need_grad;
  a.lse = lse; a.target_logit = target_logit; a.ce = ce; a.entropy = entropy; a.argmax = argmax;
  a.cew_out = cew_out; a.loss = loss; a.metrics = metrics; a.dx = dx; a.top_logit = top_logit;
  a.overflow = overflow;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes; a.stream = stream;
  return step_impl(a);
}

size_t esep_head_train_workspace_bytes(int64_t n, int64_t h, int64_t v, int dtype) {
  return esep_head_step_workspace_bytes(n, h, v, dtype, 1);
}

int esep_head_train(const void* x, const void* w, const void* w_bf16, const int64_t* target,
                    const float* ce_weight, int64_t n, int64_t h, int64_t v, int dtype, float* lse,
                    float* target_logit, float* ce, float* entropy, int64_t* argmax,
                    float* cew_out, float* loss, float* metrics, float* dx, int* overflow,
                    void* workspace, size_t workspace_bytes, void* stream) {
  if (target == nullptr || ce_weight == nullptr || overflow == nullptr) return ESEP_ERR_BAD_ARG;
  // the four scalars of the older interface are the first four of the step's eight
  float* m8 = nullptr;
  if (metrics != nullptr) {
    if (workspace == nullptr || workspace_bytes < kAlign) return ESEP_ERR_WORKSPACE;
    m8 = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + 128);   // status block
  }
  const int st = esep_head_step(x, dtype, w, w_bf16, dtype, n, h, v, target, ce_weight, nullptr,
                                nullptr, 0, 1, lse, target_logit, ce, entropy, argmax, cew_out, loss,
                                m8, dx, nullptr, overflow, workspace, workspace_bytes, stream);
  if (st != ESEP_OK || metrics == nullptr) return st;
  return cudaMemcpyAsync(metrics, m8, ESEP_METRIC_SCALARS * sizeof(float),
                         cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? ESEP_OK
             : ESEP_ERR_CUDA;
}

int esep_head_vp_prepare(const int64_t* target, int64_t n, int64_t vocab_offset, int64_t v_local,
                         int64_t v_global, int64_t* local_target, float* unit_weight,
                         void* stream) {
  if (target == nullptr || local_target == nullptr || unit_weight == nullptr || n <= 0 ||
      n > (1 << 30) || v_local <= 0 || v_global <= 0 || vocab_offset < 0)
    return ESEP_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  head_vp_prepare_kernel<<<div_up(n, 256), 256, 0, s>>>(
      static_cast<int>(n), v_global, vocab_offset, v_local,
      reinterpret_cast<const long long*>(target), reinterpret_cast<long long*>(local_target),
      unit_weight);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_vp_pack(const float* lse, const float* entropy, const float* top_logit,
                      const float* target_logit, const int64_t* argmax_local,
                      const int64_t* target, int64_t n, int64_t vocab_offset, int64_t v_local,
                      int64_t v_global, float* record, void* stream) {
  if (lse == nullptr || entropy == nullptr || top_logit == nullptr || target_logit == nullptr ||
      argmax_local == nullptr || target == nullptr || record == nullptr || n <= 0 ||
      n > (1 << 30))
    return ESEP_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  head_vp_pack_kernel<<<div_up(n, 256), 256, 0, s>>>(
      static_cast<int>(n), v_global, vocab_offset, v_local,
      reinterpret_cast<const long long*>(target), lse, entropy, top_logit, target_logit,
      reinterpret_cast<const long long*>(argmax_local), record);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_vp_combine(const float* records, int n_records, int my_record,
                         const int64_t* target, const float* ce_weight, const void* w_shard,
                         int64_t n, int64_t h, int64_t v_local, int64_t vocab_offset,
                         int64_t v_global, int dtype, float* dx, float* lse, float* target_logit,
                         float* ce, float* entropy, int64_t* argmax, float* cew_out, float* loss,
                         float* metrics, void* stream) {
  if (records == nullptr || target == nullptr || ce_weight == nullptr || w_shard == nullptr ||
      dx == nullptr || lse == nullptr || target_logit == nullptr || ce == nullptr ||
      entropy == nullptr || argmax == nullptr || cew_out == nullptr || loss == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (n <= 0 || n > (1 << 30) || h <= 0 || h % 8 != 0 || v_local <= 0 || v_global <= 0 ||
      n_records <= 0 || my_record < 0 || my_record >= n_records)
    return ESEP_ERR_BAD_ARG;
  if (dtype != ESEP_DTYPE_F16 && dtype != ESEP_DTYPE_BF16) return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(dx) & 15u) || (reinterpret_cast<uintptr_t>(w_shard) & 15u))
    return ESEP_ERR_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  VpCombineParams q = {};
  q.n = static_cast<int>(n);
  q.h = static_cast<int>(h);
  q.k_parts = n_records;
  q.me = my_record;
  q.v_global = v_global;
  q.vocab_offset = vocab_offset;
  q.v_local = v_local;
  q.records = records;
  q.target = reinterpret_cast<const long long*>(target);
  q.ce_weight = ce_weight;
  q.w_shard = w_shard;
  q.dx = dx;
  q.lse = lse; q.tlogit = target_logit; q.ce = ce; q.ent = entropy; q.cew_out = cew_out;
  q.amax = reinterpret_cast<long long*>(argmax);
  if (dtype == ESEP_DTYPE_F16)
    head_vp_combine_kernel<0><<<static_cast<unsigned>(n), 128, 0, s>>>(q);
  else
    head_vp_combine_kernel<1><<<static_cast<unsigned>(n), 128, 0, s>>>(q);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  head_scalars_kernel<<<1, 1024, 0, s>>>(q.n, v_global, ce, cew_out, entropy,
                                         reinterpret_cast<const long long*>(argmax),
                                         reinterpret_cast<const long long*>(target), nullptr, loss,
                                         metrics);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_head_grad_scale(const float* dx, const float* grad_loss, int64_t count, int out_dtype,
                         void* out, void* stream) {
  if (dx == nullptr || grad_loss == nullptr || out == nullptr || count < 0 || count % 4 != 0)
    return ESEP_ERR_BAD_ARG;
  if (out_dtype != ESEP_DTYPE_F16 && out_dtype != ESEP_DTYPE_BF16 && out_dtype != ESEP_DTYPE_F32)
    return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(dx) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return ESEP_ERR_ALIGNMENT;
  if (count == 0) return ESEP_OK;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long n4 = count / 4;
  const unsigned grid = static_cast<unsigned>(std::min<long long>((n4 + 255) / 256, 8LL * d->sm_count));
  const float4* src = reinterpret_cast<const float4*>(dx);
  if (out_dtype == ESEP_DTYPE_F16) head_grad_scale_kernel<0><<<grid, 256, 0, s>>>(src, grad_loss, n4, out);
  else if (out_dtype == ESEP_DTYPE_BF16) head_grad_scale_kernel<1><<<grid, 256, 0, s>>>(src, grad_loss, n4, out);
  else head_grad_scale_kernel<2><<<grid, 256, 0, s>>>(src, grad_loss, n4, out);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

// ---- the shared fp16 weight format (head_weight.cuh) ------------------------------------------
int esep_weight_fixup_scan(const float* w32, void* w16, int cast, int64_t v, int64_t h,
                           int32_t* row_start, int64_t* stats, void* stream) {
  if (w32 == nullptr || w16 == nullptr || row_start == nullptr || stats == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (v <= 0 || h <= 0 || h % 8 != 0 || v >= (1LL << 31) - 1 || h > (1 << 20))
    return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(w32) & 15u) || (reinterpret_cast<uintptr_t>(w16) & 15u))
    return ESEP_ERR_ALIGNMENT;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned row_blocks = static_cast<unsigned>((v + 1023) / 1024);
  long long* st64 = reinterpret_cast<long long*>(stats);
  if (cudaMemsetAsync(st64, 0, (3 + static_cast<size_t>(row_blocks)) * sizeof(long long), s) !=
      cudaSuccess)
    return ESEP_ERR_CUDA;
  const unsigned rows_grid = static_cast<unsigned>(v);
  if (cast)
    head_w16_scan_kernel<true><<<rows_grid, 128, 0, s>>>(w32, static_cast<__half*>(w16),
                                                         static_cast<int>(v), static_cast<int>(h),
                                                         row_start, st64);
  else
    head_w16_scan_kernel<false><<<rows_grid, 128, 0, s>>>(w32, static_cast<__half*>(w16),
                                                          static_cast<int>(v), static_cast<int>(h),
                                                          row_start, st64);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  head_w16_offsets_kernel<<<row_blocks, 1024, 0, s>>>(row_start, static_cast<int>(v), st64);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(2);
  return ESEP_OK;
}

int esep_weight_fixup_fill(const float* w32, const void* w16, int64_t v, int64_t h,
                           const int32_t* row_start, int64_t* flat_idx, float* flat_val,
                           void* stream) {
  if (w32 == nullptr || w16 == nullptr || row_start == nullptr || flat_idx == nullptr ||
      flat_val == nullptr)
    return ESEP_ERR_BAD_ARG;
  if (v <= 0 || h <= 0 || h % 8 != 0 || v >= (1LL << 31) - 1 || h > (1 << 20))
    return ESEP_ERR_BAD_ARG;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  head_w16_fill_kernel<<<static_cast<unsigned>(v), 128, 0, s>>>(w32, static_cast<const __half*>(w16),
                                            static_cast<int>(v), static_cast<int>(h), row_start,
                                            reinterpret_cast<long long*>(flat_idx), flat_val);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_embed_rows(const void* w16, const int64_t* ids, int64_t n, int64_t v, int64_t h,
                    const int32_t* row_start, const int64_t* flat_idx, const float* flat_val,
                    float* out, int* status, void* stream) {
  if (ids == nullptr || out == nullptr || n < 0 || n > (1LL << 30)) return ESEP_ERR_BAD_ARG;
  if (v <= 0 || h <= 0 || h % 8 != 0 || v >= (1LL << 31) - 1 || h > (1 << 20))
    return ESEP_ERR_BAD_ARG;
  if (row_start != nullptr && (flat_idx == nullptr || flat_val == nullptr)) return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(w16) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return ESEP_ERR_ALIGNMENT;
  if (n == 0 || (w16 == nullptr && row_start == nullptr)) return ESEP_OK;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  head_embed_rows_kernel<<<static_cast<unsigned>(n), 128, 0, s>>>(
      static_cast<const __half*>(w16), reinterpret_cast<const long long*>(ids),
      static_cast<int>(v), static_cast<int>(h), row_start,
      reinterpret_cast<const long long*>(flat_idx), flat_val, out, status);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  return ESEP_OK;
}

int esep_weight_exact(const void* w16, int64_t v, int64_t h, int64_t count,
                      const int64_t* flat_idx, const float* flat_val, float* out, void* stream) {
  if (w16 == nullptr || out == nullptr || count < 0) return ESEP_ERR_BAD_ARG;
  if (v <= 0 || h <= 0 || h % 8 != 0 || v >= (1LL << 31) - 1 || h > (1 << 20))
    return ESEP_ERR_BAD_ARG;
  if (count > 0 && (flat_idx == nullptr || flat_val == nullptr)) return ESEP_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(w16) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return ESEP_ERR_ALIGNMENT;
  const DeviceInfo* d = nullptr;
  const int st = current_device_info(&d);
  if (st != ESEP_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t n8 = static_cast<size_t>(v) * h / 8;
  if ((n8 + 1023) / 1024 > 0x7fffffffull) return ESEP_ERR_BAD_ARG;
  const unsigned grid = static_cast<unsigned>((n8 + 1023) / 1024);
  head_w16_upcast_kernel<<<grid, 256, 0, s>>>(static_cast<const __half*>(w16), n8, out);
  if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
  g_launches.fetch_add(1);
  if (count > 0) {
    head_w16_restore_kernel<<<static_cast<unsigned>((count + 255) / 256), 256, 0, s>>>(
        reinterpret_cast<const long long*>(flat_idx), flat_val, count, out);
    if (cudaGetLastError() != cudaSuccess) return ESEP_ERR_CUDA;
    g_launches.fetch_add(1);
  }
  return ESEP_OK;
}

int esep_head_step_uses_stored_logits(int64_t m, int64_t h, int64_t v, int dtype, int need_grad) {
  if (m <= 0 || h <= 0 || v <= 0 || h % 8 != 0) return 0;
  if (dtype != ESEP_DTYPE_F16 && dtype != ESEP_DTYPE_BF16) return 0;
  const DeviceInfo* d = nullptr;
  if (current_device_info(&d) != ESEP_OK) return 0;
  StepLayout t;
  if (step_layout(m, h, v, need_grad != 0, d, &t) != ESEP_OK) return 0;
  return t.stored ? (t.direct ? 2 : 1) : 0;
}

int esep_head_step_path_taken(const void* workspace, void* stream, int* out_stored) {
  if (workspace == nullptr || out_stored == nullptr) return ESEP_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int v = 0;
  // the step keeps its row counts at byte 64 of the workspace (CNT_*)
  if (cudaMemcpyAsync(&v, static_cast<const uint8_t*>(workspace) + 64 + CNT_STORED * sizeof(int),
                      sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    cudaGetLastError();
    return ESEP_ERR_CUDA;
  }
  *out_stored = v;
  return ESEP_OK;
}

int esep_head_set_training_path(int path) {
  if (path < 0 || path > 3) return ESEP_ERR_BAD_ARG;
  return g_training_path.exchange(path);
}

int esep_head_debug_counters(long long* out, int n) {
  if (out == nullptr || n < 2) return ESEP_ERR_BAD_ARG;
  out[0] = g_init_calls.load();
  out[1] = g_tmap_encodes.load();
  if (n >= 3) out[2] = g_launches.load();
  if (n >= 4) out[3] = g_wide_launches.load();
  if (n >= 5) out[4] = g_dx_launches.load();
  return ESEP_OK;
}

}  // extern "C"
