// Host-side helpers shared by the extension's translation units: TMA descriptor encoding through
// the driver entry point (no link-time dependency on libcuda), per-device scratch/status
// buffers, and argument checks.
#pragma once
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <torch/extension.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

namespace b200 {

#define B200_CUDA_CHECK(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    TORCH_CHECK(_e == cudaSuccess, #expr " failed: ", cudaGetErrorString(_e));             \
  } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    TORCH_CHECK(e == cudaSuccess && p != nullptr && qres == cudaDriverEntryPointSuccess,
                "cuTensorMapEncodeTiled is not available from the CUDA driver");
    fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 tensor map with 128-byte swizzle.  `inner` elements are contiguous, rows are
// `ld_elems` apart.  The innermost box extent must be 64 elements (128 bytes).
inline void encode_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                                uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer) {
  TORCH_CHECK((reinterpret_cast<uintptr_t>(base) & 15) == 0, "TMA base must be 16-byte aligned");
  TORCH_CHECK((ld_elems * 2) % 16 == 0, "TMA row pitch must be a multiple of 16 bytes");
  TORCH_CHECK(box_inner * 2 == 128, "inner box must span 128 bytes");
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld_elems * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = get_encode_tiled()(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code ", static_cast<int>(r));
}

// Number of kernels of this extension launched so far in this process (all devices).
inline std::atomic<long long>& launch_counter() {
  static std::atomic<long long> n{0};
  return n;
}
inline void count_launch(int n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }

// Per-device persistent buffers: scratch for split-K partials and the status word.
struct DeviceState {
  at::Tensor scratch;   // fp32
  at::Tensor status;    // int32[1]
};

inline DeviceState& device_state(int dev) {
  static std::unordered_map<int, DeviceState> states;
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  auto it = states.find(dev);
  if (it == states.end()) {
    DeviceState s;
    auto opt_i = at::TensorOptions().dtype(at::kInt).device(at::kCUDA, dev);
    s.status = at::zeros({1}, opt_i);
    it = states.emplace(dev, std::move(s)).first;
  }
  return it->second;
}

inline float* ensure_scratch(int dev, size_t nfloats) {
  DeviceState& s = device_state(dev);
  if (!s.scratch.defined() || static_cast<size_t>(s.scratch.numel()) < nfloats) {
    size_t n = nfloats < (1u << 22) ? (1u << 22) : nfloats;
    s.scratch = at::empty({static_cast<int64_t>(n)},
                          at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, dev));
  }
  return s.scratch.data_ptr<float>();
}

}  // namespace b200
