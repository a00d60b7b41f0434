// Per-device state of the int4tc_b200 library: cached properties, the device status word that
// bounded waits write to, and the tensor-map cache.
#include "gemm.cuh"
#include <mutex>
#include <vector>
#include <cstring>

namespace i4tc {

static constexpr int kMaxDevices = 64;
static DeviceInfo g_info[kMaxDevices];
static std::mutex g_mutex;

int device_info(int device, const DeviceInfo** out) {
  I4TC_REQUIRE(device >= 0 && device < kMaxDevices, I4TC_EINVAL, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceInfo& d = g_info[device];
  if (!d.valid) {
    DeviceGuard guard(device);
    I4TC_CUDA(guard.err);
    I4TC_CUDA(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, device));
    I4TC_CUDA(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, device));
    I4TC_CUDA(cudaDeviceGetAttribute(&d.cc_minor, cudaDevAttrComputeCapabilityMinor, device));
    I4TC_CUDA(cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, device));
    I4TC_CUDA(cudaMalloc(&d.status, sizeof(unsigned int)));
    I4TC_CUDA(cudaMemset(d.status, 0, sizeof(unsigned int)));
    d.valid = true;
  }
  *out = &d;
  return I4TC_OK;
}

// ---- split-K workspaces ------------------------------------------------------------------
// One grow-only arena per (device, stream): calls on different streams never share partial sums, and a pointer
// that was handed out stays valid until i4tc_release_workspaces or process exit -- a CUDA graph captured earlier,
// or a launch still in flight, may hold it.  Growth allocates a new, larger buffer and keeps the old ones.
struct WsArena {
  int device;
  cudaStream_t stream;
  float* cur = nullptr;
  size_t cur_bytes = 0;
  std::vector<void*> retired;   // smaller buffers handed out earlier
};
static std::vector<WsArena> g_arenas;
static constexpr size_t kWsMinBytes = 16u << 20;

static int arena_reserve(int device, cudaStream_t stream, size_t bytes, float** out) {
  WsArena* a = nullptr;
  for (auto& x : g_arenas)
    if (x.device == device && x.stream == stream) a = &x;
  if (a == nullptr) {
    g_arenas.push_back(WsArena{device, stream});
    a = &g_arenas.back();
  }
  if (a->cur_bytes < bytes) {
    DeviceGuard guard(device);
    I4TC_CUDA(guard.err);
    size_t want = bytes < kWsMinBytes ? kWsMinBytes : bytes;
    if (want < 2 * a->cur_bytes) want = 2 * a->cur_bytes;   // geometric growth bounds what the retired buffers hold
    void* p = nullptr;
    const cudaError_t e = cudaMalloc(&p, want);
    if (e != cudaSuccess) {
      cudaGetLastError();
      return fail(I4TC_EWORKSPACE,
                  "the split-K workspace of this stream holds %zu bytes and %zu are needed, but cudaMalloc failed (%s); "
                  "reserve it beforehand with i4tc_reserve_workspace (outside stream capture)",
                  a->cur_bytes, bytes, cudaGetErrorName(e));
    }
    if (a->cur) a->retired.push_back(a->cur);
    a->cur = static_cast<float*>(p);
    a->cur_bytes = want;
  }
  if (out) *out = a->cur;
  return I4TC_OK;
}

int split_workspace(int device, cudaStream_t stream, size_t bytes, float** out) {
  const DeviceInfo* cinfo;
  if (int rc = device_info(device, &cinfo)) return rc;
  std::lock_guard<std::mutex> lock(g_mutex);
  return arena_reserve(device, stream, bytes, out);
}

// ---- tensor maps -------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct MapKey {
  const void* base;
  long long rows, extent;
  int box_rows, rowmajor, device;   // rowmajor: 0 = group-major packed, 1 = row-major packed, 2 = row-major int8 (swizzled)
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && extent == o.extent && box_rows == o.box_rows &&
           rowmajor == o.rowmajor && device == o.device;
  }
};
struct MapEntry {
  MapKey key;
  CUtensorMap map;
  bool used = false;
};
static constexpr int kMapCache = 256;
static MapEntry g_maps[kMapCache];
static int g_map_next = 0;

int get_tensor_map(int device, const void* base, bool rowmajor, long long rows, long long extent, int box_rows,
                   CUtensorMap* out) {
  I4TC_REQUIRE(aligned_to(base, 16), I4TC_EALIGN, "packed operand must be 16-byte aligned");
  I4TC_REQUIRE(rows > 0 && extent > 0, I4TC_EINVAL, "empty operand");
  I4TC_REQUIRE(rows < (1ll << 31), I4TC_EINVAL, "operand has too many rows");
  MapKey key{base, rows, extent, box_rows, rowmajor ? 1 : 0, device};
  std::lock_guard<std::mutex> lock(g_mutex);
  for (int i = 0; i < kMapCache; ++i)
    if (g_maps[i].used && g_maps[i].key == key) {
      *out = g_maps[i].map;
      return I4TC_OK;
    }
  EncodeTiledFn fn = encode_fn();
  I4TC_REQUIRE(fn != nullptr, I4TC_EDEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap m;
  CUresult r;
  if (rowmajor) {
    // [rows, row_bytes] bytes; a box is 64 bytes (one K group) by box_rows rows
    I4TC_REQUIRE(extent % 16 == 0, I4TC_EALIGN, "packed row length must be a multiple of 16 bytes");
    cuuint64_t dims[2] = {(cuuint64_t)extent, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)extent};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    // [slabs, rows, 64] bytes
    cuuint64_t dims[3] = {64u, (cuuint64_t)rows, (cuuint64_t)extent};
    cuuint64_t strides[2] = {64u, (cuuint64_t)rows * 64u};
    cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  I4TC_REQUIRE(r == CUDA_SUCCESS, I4TC_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  MapEntry& e = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % kMapCache;
  e.key = key;
  e.map = m;
  e.used = true;
  *out = m;
  return I4TC_OK;
}

int get_tensor_map_i8(int device, const void* base, long long rows, long long K, int box_rows, CUtensorMap* out) {
  I4TC_REQUIRE(aligned_to(base, 16), I4TC_EALIGN, "int8 operand must be 16-byte aligned");
  I4TC_REQUIRE(rows > 0 && K > 0 && rows < (1ll << 31), I4TC_EINVAL, "bad operand shape");
  I4TC_REQUIRE(K % 16 == 0, I4TC_EALIGN, "K must be a multiple of 16 for int8 operands");
  MapKey key{base, rows, K, box_rows, 2, device};
  std::lock_guard<std::mutex> lock(g_mutex);
  for (int i = 0; i < kMapCache; ++i)
    if (g_maps[i].used && g_maps[i].key == key) {
      *out = g_maps[i].map;
      return I4TC_OK;
    }
  EncodeTiledFn fn = encode_fn();
  I4TC_REQUIRE(fn != nullptr, I4TC_EDEVICE, "cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap m;
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  const CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  I4TC_REQUIRE(r == CUDA_SUCCESS, I4TC_EINVAL, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  MapEntry& e = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % kMapCache;
  e.key = key;
  e.map = m;
  e.used = true;
  *out = m;
  return I4TC_OK;
}

}  // namespace i4tc

using namespace i4tc;

extern "C" int i4tc_version(void) { return 100; }

extern "C" const char* i4tc_last_error(void) { return err_buf(); }

extern "C" int i4tc_sm_count(int device) {
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc < 0 ? rc : -rc;
  return info->sm_count;
}

extern "C" int i4tc_reserve_workspace(int device, void* stream, int64_t bytes) {
  I4TC_REQUIRE(bytes >= 0, I4TC_EINVAL, "negative size");
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  std::lock_guard<std::mutex> lock(g_mutex);
  return arena_reserve(device, static_cast<cudaStream_t>(stream), (size_t)bytes, nullptr);
}

extern "C" int64_t i4tc_workspace_bytes(int device, void* stream) {
  std::lock_guard<std::mutex> lock(g_mutex);
  for (auto& a : g_arenas)
    if (a.device == device && a.stream == static_cast<cudaStream_t>(stream)) return (int64_t)a.cur_bytes;
  return 0;
}

extern "C" int i4tc_release_workspaces(int device) {
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  I4TC_CUDA(cudaDeviceSynchronize());   // nothing in flight may still use a buffer
  for (auto it = g_arenas.begin(); it != g_arenas.end();) {
    if (it->device != device) { ++it; continue; }
    for (void* p : it->retired) cudaFree(p);
    if (it->cur) cudaFree(it->cur);
    it = g_arenas.erase(it);
  }
  return I4TC_OK;
}

extern "C" int i4tc_check_status(int device, void* stream) {
  const DeviceInfo* info;
  if (int rc = device_info(device, &info)) return rc;
  DeviceGuard guard(device);
  I4TC_CUDA(guard.err);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned int h = 0;
  I4TC_CUDA(cudaMemcpyAsync(&h, info->status, sizeof(h), cudaMemcpyDeviceToHost, st));
  I4TC_CUDA(cudaStreamSynchronize(st));
  if (h != 0) {
    I4TC_CUDA(cudaMemsetAsync(info->status, 0, sizeof(unsigned int), st));
    I4TC_CUDA(cudaStreamSynchronize(st));
    return fail(I4TC_EKERNEL, "a kernel gave up on a bounded wait (status word 0x%x)", h);
  }
  return I4TC_OK;
}
