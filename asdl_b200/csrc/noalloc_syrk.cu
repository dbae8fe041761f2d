// Allocation-free variant of the split-K SYRK (see noalloc_api.h for the contract).
//
// The kernels are the ones of umma_gemm.cuh, compiled a second time into this translation unit
// under different names so that the scratch pointer handed to them can come from the static
// device array below instead of from an allocator.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <mutex>

#define umma_gemm_kernel umma_gemm_kernel_noalloc
#define splitk_reduce_kernel splitk_reduce_kernel_noalloc
#include "umma_gemm.cuh"
#undef umma_gemm_kernel
#undef splitk_reduce_kernel

#include "noalloc_api.h"

namespace {

constexpr size_t kScratchFloats = ASDL_B200_NOALLOC_SCRATCH_BYTES / sizeof(float);

// Scratch for the split-K partial tiles.  In host code this name is only a stand-in for the
// symbol: its device address has to be asked for with cudaGetSymbolAddress (done once per device
// in device_slot()).  Device code may use the array directly.
static __device__ __align__(256) float g_noalloc_scratch[kScratchFloats];
static __device__ int g_noalloc_status;

constexpr int kMaxDevices = 64;
constexpr long long kMaxRows = 0x7fffffffll - 64;  // rows + 63 must fit a signed 32-bit integer
constexpr long long kMaxN = 1 << 16;               // 512 tile rows: the tile count stays far below 2^31

struct DeviceSlot {
  bool ready = false;
  float* scratch = nullptr;
  int* status = nullptr;
  int sm_count = 0;
};

DeviceSlot g_slots[kMaxDevices];
std::mutex g_slot_mutex;

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

int fail(char* err, int err_len, int code, const char* fmt, long long a = 0, long long b = 0) {
  if (err != nullptr && err_len > 0) std::snprintf(err, static_cast<size_t>(err_len), fmt, a, b);
  return code;
}

// One-time set-up for the current device: device addresses of the static arrays, the kernel's
// shared-memory limit and the SM count.  Runs with that device current.
int device_slot(int dev, DeviceSlot** out, char* err, int err_len) {
  if (dev < 0 || dev >= kMaxDevices) return fail(err, err_len, 10, "device index %lld is out of range", dev);
  std::lock_guard<std::mutex> guard(g_slot_mutex);
  DeviceSlot& slot = g_slots[dev];
  if (!slot.ready) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(err, err_len, 11, "cudaGetSymbolAddress(scratch) failed with CUDA error %lld", e);
    slot.scratch = static_cast<float*>(p);
    e = cudaGetSymbolAddress(&p, g_noalloc_status);
    if (e != cudaSuccess || p == nullptr)
      return fail(err, err_len, 12, "cudaGetSymbolAddress(status) failed with CUDA error %lld", e);
    slot.status = static_cast<int*>(p);
    e = cudaFuncSetAttribute(b200::umma_gemm_kernel_noalloc,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, b200::G_SMEM_BYTES);
    if (e != cudaSuccess)
      return fail(err, err_len, 13, "cudaFuncSetAttribute failed with CUDA error %lld", e);
    e = cudaDeviceGetAttribute(&slot.sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || slot.sm_count <= 0)
      return fail(err, err_len, 14, "cudaDeviceGetAttribute failed with CUDA error %lld", e);
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess || fn == nullptr || q != cudaDriverEntryPointSuccess)
        return fail(err, err_len, 15, "cuTensorMapEncodeTiled is not available (CUDA error %lld)", e);
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    slot.ready = true;
  }
  *out = &slot;
  return 0;
}

}  // namespace

extern "C" int asdl_b200_syrk_bf16_noalloc(const void* x, long long rows, int n, long long ldx,
                                           float* c, int ldc, float alpha, float beta, int nsplit,
                                           void* stream, char* err, int err_len) {
  using namespace b200;
  if (x == nullptr || c == nullptr) return fail(err, err_len, 1, "x and c must not be null");
  if (rows <= 0 || n <= 0) return fail(err, err_len, 2, "rows (%lld) and n (%lld) must be positive", rows, n);
  if (ldx < n || (ldx % 8) != 0)
    return fail(err, err_len, 3, "ldx (%lld) must be >= n (%lld) and a multiple of 8", ldx, n);
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return fail(err, err_len, 4, "x must be 16-byte aligned");
  if (ldc < n) return fail(err, err_len, 5, "ldc (%lld) must be >= n (%lld)", ldc, n);
  if (nsplit < 0) return fail(err, err_len, 6, "nsplit (%lld) must be >= 0", nsplit);
  // the epilogue reads and writes C with 16-byte vectors whenever the row pitch allows it
  if ((ldc & 3) == 0 && (reinterpret_cast<uintptr_t>(c) & 15) != 0)
    return fail(err, err_len, 17, "c must be 16-byte aligned when ldc (%lld) is a multiple of 4", ldc);
  if ((reinterpret_cast<uintptr_t>(c) & 3) != 0) return fail(err, err_len, 17, "c must be 4-byte aligned");
  // the kernel keeps the row count and the tile arithmetic in 32-bit integers
  if (rows > kMaxRows) return fail(err, err_len, 18, "rows (%lld) exceeds the supported maximum (%lld)", rows, kMaxRows);
  if (n > kMaxN) return fail(err, err_len, 19, "n (%lld) exceeds the supported maximum (%lld)", n, kMaxN);

  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, err_len, 7, "cudaGetDevice failed with CUDA error %lld", e);
  DeviceSlot* slot = nullptr;
  if (int rc = device_slot(dev, &slot, err, err_len)) return rc;

  GemmProblem P;
  std::memset(&P, 0, sizeof(P));
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ldx) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(G_BK)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = g_encode(&P.tmA[0], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(x), dims,
                        strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(err, err_len, 8, "cuTensorMapEncodeTiled failed with code %lld", r);
  P.tmB[0] = P.tmA[0];
  P.C = c;
  P.Cin = c;
  P.ldc = ldc;
  P.status = slot->status;
  P.M = P.N = n;
  P.K = static_cast<int>(rows);
  P.nseg = 1;
  P.alpha = alpha;
  P.beta = beta;
  P.flags = GF_SYM | GF_SAME_AB;
  P.tiles_m = P.tiles_n = (n + G_BM - 1) / G_BM;
  P.ntiles = P.tiles_m * (P.tiles_m + 1) / 2;
  const int kb_total = static_cast<int>((rows + G_BK - 1) / G_BK);
  const size_t tile_floats = static_cast<size_t>(G_BM) * G_BN;
  if (nsplit == 0) {  // same rule as the allocating entry point, capped by the scratch capacity
    nsplit = (2 * slot->sm_count) / P.ntiles;
    if (nsplit > kb_total / 8) nsplit = kb_total / 8;
    if (nsplit > 32) nsplit = 32;
    const size_t cap = kScratchFloats / (tile_floats * static_cast<size_t>(P.ntiles));
    if (static_cast<size_t>(nsplit) > cap) nsplit = static_cast<int>(cap);
  }
  if (nsplit > kb_total) nsplit = kb_total;
  if (nsplit < 1) nsplit = 1;
  P.nsplit = nsplit;
  if (nsplit > 1) {
    const size_t need = tile_floats * static_cast<size_t>(P.ntiles) * static_cast<size_t>(nsplit);
    if (need > kScratchFloats)
      return fail(err, err_len, 9,
                  "request needs %lld bytes of scratch but the built-in buffer holds %lld; use a smaller nsplit",
                  static_cast<long long>(need * sizeof(float)),
                  static_cast<long long>(ASDL_B200_NOALLOC_SCRATCH_BYTES));
    P.ws = slot->scratch;  // every (tile, split) slice is fully rewritten before it is read
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  umma_gemm_kernel_noalloc<<<dim3(P.ntiles, P.nsplit, 1), G_THREADS, G_SMEM_BYTES, s>>>(P, nullptr, nullptr);
  if (nsplit > 1)
    splitk_reduce_kernel_noalloc<<<dim3(P.ntiles, 16, 1), 256, 0, s>>>(P, nullptr, nullptr);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(err, err_len, 16, "kernel launch failed with CUDA error %lld", e);
  return 0;
}

// Reads the status word that the kernels of this entry point write when one of their bounded
// waits ran out (the b200::ERR_* codes), stores it in *code and clears it.  Waits for the work
// already enqueued on the current device; allocates nothing.
extern "C" int asdl_b200_noalloc_status(int* code) {
  if (code == nullptr) return 1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 7;
  DeviceSlot* slot = nullptr;
  if (int rc = device_slot(dev, &slot, nullptr, 0)) return rc;
  int value = 0;
  if (cudaMemcpyFromSymbol(&value, g_noalloc_status, sizeof(int)) != cudaSuccess) return 20;
  if (value != 0) {
    const int zero = 0;
    if (cudaMemcpyToSymbol(g_noalloc_status, &zero, sizeof(int)) != cudaSuccess) return 21;
  }
  *code = value;
  return 0;
}
