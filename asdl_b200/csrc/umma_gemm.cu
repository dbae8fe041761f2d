// Host launcher for the tcgen05 TN-GEMM / SYRK kernel (see umma_gemm.cuh).
#include "host_utils.h"
#include "umma_gemm.cuh"

#include <unordered_map>

namespace b200 {

namespace {

struct Ring {
  size_t off = 0;
};
Ring g_scratch_ring[16];

void check_operand(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2, name,
              " must be a 2-D CUDA bf16 tensor");
  TORCH_CHECK(t.stride(1) == 1, name, " must have unit stride in its last dimension");
  TORCH_CHECK((t.stride(0) * 2) % 16 == 0, name, " row pitch must be a multiple of 16 bytes");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name,
              " must be 16-byte aligned");
}

bool g_attr_set = false;

}  // namespace

// Fills the scalar fields of a problem and encodes its tensor maps.
void gemm_fill_problem(GemmProblem& P, const std::vector<at::Tensor>& a_segs,
                       const std::vector<at::Tensor>& b_segs, bool a_kmajor, bool b_kmajor,
                       const c10::optional<at::Tensor>& C, double alpha, double beta, bool sym,
                       const c10::optional<at::Tensor>& out_hi,
                       const c10::optional<at::Tensor>& out_lo, int64_t nsplit_req, int n_sms,
                       bool allow_no_output = false) {
  const int nseg = static_cast<int>(a_segs.size());
  TORCH_CHECK(nseg >= 1 && nseg <= 3 && b_segs.size() == a_segs.size(),
              "between 1 and 3 operand segments are supported");
  std::memset(&P, 0, sizeof(P));
  const at::Tensor& a0 = a_segs[0];
  const at::Tensor& b0 = b_segs[0];
  const int64_t M = a_kmajor ? a0.size(0) : a0.size(1);
  const int64_t K = a_kmajor ? a0.size(1) : a0.size(0);
  const int64_t N = b_kmajor ? b0.size(0) : b0.size(1);
  const int64_t Kb = b_kmajor ? b0.size(1) : b0.size(0);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  for (int s = 0; s < nseg; ++s) {
    check_operand(a_segs[s], "A");
    check_operand(b_segs[s], "B");
    TORCH_CHECK(a_segs[s].sizes() == a0.sizes() && b_segs[s].sizes() == b0.sizes(),
                "all segments must have the same shape");
    if (a_kmajor)
      encode_tmap_bf16_2d(&P.tmA[s], a_segs[s].data_ptr(), K, M, a_segs[s].stride(0), 64, G_BM);
    else
      encode_tmap_bf16_2d(&P.tmA[s], a_segs[s].data_ptr(), M, K, a_segs[s].stride(0), 64, G_BK);
    if (b_kmajor)
      encode_tmap_bf16_2d(&P.tmB[s], b_segs[s].data_ptr(), K, N, b_segs[s].stride(0), 64, G_BN);
    else
      encode_tmap_bf16_2d(&P.tmB[s], b_segs[s].data_ptr(), N, K, b_segs[s].stride(0), 64, G_BK);
  }
  bool same_ab = sym && a_kmajor == b_kmajor;
  for (int s = 0; s < nseg && same_ab; ++s)
    same_ab = a_segs[s].data_ptr() == b_segs[s].data_ptr() &&
              a_segs[s].stride(0) == b_segs[s].stride(0);
  if (sym) TORCH_CHECK(M == N, "symmetric mode needs a square output");

  P.M = static_cast<int>(M);
  P.N = static_cast<int>(N);
  P.K = static_cast<int>(K);
  P.nseg = nseg;
  P.alpha = static_cast<float>(alpha);
  P.beta = static_cast<float>(beta);
  P.flags = (sym ? GF_SYM : 0) | (a_kmajor ? GF_A_KMAJOR : 0) | (b_kmajor ? GF_B_KMAJOR : 0) |
            (same_ab ? GF_SAME_AB : 0);
  if (C.has_value()) {
    const at::Tensor& c = *C;
    TORCH_CHECK(c.is_cuda() && c.scalar_type() == at::kFloat && c.dim() == 2 && c.stride(1) == 1 &&
                    c.size(0) == M && c.size(1) == N,
                "C must be a [M, N] fp32 CUDA tensor with unit column stride");
    P.C = c.data_ptr<float>();
    P.Cin = P.C;
    P.ldc = static_cast<int>(c.stride(0));
  } else {
    TORCH_CHECK(beta == 0.0, "beta needs C");
  }
  if (out_hi.has_value()) {
    const at::Tensor& h = *out_hi;
    TORCH_CHECK(h.is_cuda() && h.scalar_type() == at::kBFloat16 && h.dim() == 2 &&
                    h.stride(1) == 1 && h.size(0) == M && h.size(1) >= N,
                "out_hi must be a [M, >=N] bf16 CUDA tensor");
    P.out_hi = reinterpret_cast<__nv_bfloat16*>(h.data_ptr());
    P.ld_out = static_cast<int>(h.stride(0));
    if (out_lo.has_value()) {
      TORCH_CHECK(out_lo->sizes() == h.sizes() && out_lo->strides() == h.strides() &&
                      out_lo->scalar_type() == at::kBFloat16,
                  "out_lo must match out_hi");
      P.out_lo = reinterpret_cast<__nv_bfloat16*>(out_lo->data_ptr());
    }
  }
  TORCH_CHECK(allow_no_output || P.C != nullptr || P.out_hi != nullptr, "no output given");

  P.tiles_m = (P.M + G_BM - 1) / G_BM;
  P.tiles_n = (P.N + G_BN - 1) / G_BN;
  P.ntiles = sym ? P.tiles_m * (P.tiles_m + 1) / 2 : P.tiles_m * P.tiles_n;
  const int kb_total = (P.K + G_BK - 1) / G_BK;
  int nsplit = static_cast<int>(nsplit_req);
  if (nsplit <= 0) {
    const int target = 2 * n_sms;
    nsplit = target / (P.ntiles > 0 ? P.ntiles : 1);
    const int max_by_k = kb_total / 8;
    if (nsplit > max_by_k) nsplit = max_by_k;
    if (nsplit > 32) nsplit = 32;
  }
  if (nsplit > kb_total) nsplit = kb_total;
  if (nsplit < 1) nsplit = 1;
  P.nsplit = nsplit;
}

void gemm_attach_scratch(GemmProblem& P, int dev) {
  DeviceState& st = device_state(dev);
  P.status = st.status.data_ptr<int>();
  const int slot = dev & 15;
  if (P.nsplit > 1 && !(P.flags & GF_ATOMIC)) {
    const size_t need = static_cast<size_t>(P.ntiles) * P.nsplit * G_BM * G_BN;
    const size_t cap_min = need * 4;
    float* base = ensure_scratch(dev, cap_min);
    const size_t cap = static_cast<size_t>(device_state(dev).scratch.numel());
    Ring& sr = g_scratch_ring[slot];
    if (sr.off + need > cap) sr.off = 0;
    P.ws = base + sr.off;
    sr.off += need;
  }
}

void gemm_launch_single(const GemmProblem& P, cudaStream_t stream) {
  if (!g_attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(umma_gemm_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES));
    g_attr_set = true;
  }
  dim3 grid(P.ntiles, P.nsplit, 1);
  umma_gemm_kernel<<<grid, G_THREADS, G_SMEM_BYTES, stream>>>(P, nullptr, nullptr);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  if (P.nsplit > 1 && !(P.flags & GF_ATOMIC)) {
    dim3 rgrid(P.ntiles, 16, 1);
    splitk_reduce_kernel<<<rgrid, 256, 0, stream>>>(P, nullptr, nullptr);
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
}

// Python entry: C = alpha * A^T B (+ beta C), optionally symmetric, optionally bf16 hi/lo outputs.
void umma_gemm(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
               bool b_kmajor, c10::optional<at::Tensor> C, double alpha, double beta, bool sym,
               c10::optional<at::Tensor> out_hi, c10::optional<at::Tensor> out_lo,
               int64_t nsplit) {
  TORCH_CHECK(!a_segs.empty(), "no operands");
  const int dev = a_segs[0].get_device();
  c10::cuda::CUDAGuard guard(dev);
  const int n_sms = at::cuda::getDeviceProperties(dev)->multiProcessorCount;
  GemmProblem P;
  gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, C, alpha, beta, sym, out_hi, out_lo,
                    nsplit, n_sms);
  gemm_attach_scratch(P, dev);
  gemm_launch_single(P, at::cuda::getCurrentCUDAStream(dev).stream());
}

// Variant whose fp32 result goes to raw device addresses - typically symmetric-memory buffers of
// this or another GPU.  `dst_ptr` receives the result (accumulated with reductions when `atomic`),
// `extra_ptrs` receive plain copies of it (non-atomic mode only).  All destinations use `ldc`.
void umma_gemm_to_ptr(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
                      bool b_kmajor, int64_t dst_ptr, int64_t ldc, double alpha, bool sym, int64_t atomic,
                      std::vector<int64_t> extra_ptrs, int64_t nsplit) {
  TORCH_CHECK(!a_segs.empty(), "no operands");
  TORCH_CHECK(dst_ptr != 0 && (dst_ptr & 15) == 0, "destination must be a 16-byte aligned device address");
  TORCH_CHECK(static_cast<int>(extra_ptrs.size()) <= G_MAX_EXTRA, "too many extra destinations");
  TORCH_CHECK(!((atomic == 1 || atomic == 2) && !extra_ptrs.empty()),
              "extra destinations are not supported in atomic mode");
  const int dev = a_segs[0].get_device();
  c10::cuda::CUDAGuard guard(dev);
  const int n_sms = at::cuda::getDeviceProperties(dev)->multiProcessorCount;
  GemmProblem P;
  // a dummy bf16 output satisfies the "some output" check; it is cleared again below
  gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, c10::nullopt, alpha, 0.0, sym,
                    c10::nullopt, c10::nullopt, nsplit, n_sms, /*allow_no_output=*/true);
  P.C = reinterpret_cast<float*>(dst_ptr);
  P.Cin = P.C;
  P.ldc = static_cast<int>(ldc);
  TORCH_CHECK(P.ldc >= P.N, "ldc is smaller than the number of columns");
  if (atomic == 1 || atomic == 2) P.flags |= GF_ATOMIC;
  if (atomic == 2 || atomic == 3) {
    TORCH_CHECK(sym, "lower-triangle output needs the symmetric mode");
    P.flags |= GF_LOWER;
  }
  P.n_extra = static_cast<int>(extra_ptrs.size());
  for (int e = 0; e < P.n_extra; ++e) {
    TORCH_CHECK((extra_ptrs[e] & 15) == 0, "destinations must be 16-byte aligned");
    P.C_extra[e] = reinterpret_cast<float*>(extra_ptrs[e]);
  }
  gemm_attach_scratch(P, dev);
  gemm_launch_single(P, at::cuda::getCurrentCUDAStream(dev).stream());
}

// ---- grouped execution ---------------------------------------------------------------------------
// A plan is a fixed list of GEMM problems whose operand addresses do not change (persistent
// buffers).  Its problem table and tile list live in device memory, so running the plan is two
// launches at most (all tiles of all problems, then the split-K reductions) with no host-side
// descriptor work - which also makes it replayable from a CUDA graph.
struct GemmPlan {
  std::vector<GemmProblem> problems;
  std::vector<std::vector<at::Tensor>> keep_alive;  // operands / outputs referenced by raw pointer
  at::Tensor d_problems, d_work, d_rwork, scratch;
  int n_work = 0, n_rwork = 0, dev = 0;
  bool finalized = false;
};

static std::unordered_map<int64_t, GemmPlan> g_plans;
static int64_t g_next_plan = 1;

int64_t gemm_plan_new() {
  const int64_t id = g_next_plan++;
  g_plans[id];
  return id;
}

void gemm_plan_free(int64_t id) { g_plans.erase(id); }

void gemm_plan_add(int64_t id, std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs,
                   bool a_kmajor, bool b_kmajor, c10::optional<at::Tensor> C, double alpha, double beta,
                   bool sym, c10::optional<at::Tensor> out_hi, c10::optional<at::Tensor> out_lo,
                   int64_t dst_ptr, int64_t ldc, bool atomic, std::vector<int64_t> extra_ptrs,
                   int64_t nsplit) {
  auto it = g_plans.find(id);
  TORCH_CHECK(it != g_plans.end() && !it->second.finalized, "unknown or finalized plan");
  GemmPlan& plan = it->second;
  TORCH_CHECK(!a_segs.empty(), "no operands");
  plan.dev = a_segs[0].get_device();
  c10::cuda::CUDAGuard guard(plan.dev);
  GemmProblem P;
  gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, C, alpha, beta, sym, out_hi, out_lo,
                    nsplit <= 0 ? 1 : nsplit, 148, /*allow_no_output=*/dst_ptr != 0);
  if (dst_ptr != 0) {
    TORCH_CHECK((dst_ptr & 15) == 0, "destination must be 16-byte aligned");
    P.C = reinterpret_cast<float*>(dst_ptr);
    P.Cin = P.C;
    P.ldc = static_cast<int>(ldc);
    TORCH_CHECK(P.ldc >= P.N, "ldc is smaller than the number of columns");
  }
  if (atomic) P.flags |= GF_ATOMIC;
  TORCH_CHECK(static_cast<int>(extra_ptrs.size()) <= G_MAX_EXTRA, "too many extra destinations");
  TORCH_CHECK(!(atomic && !extra_ptrs.empty()), "extra destinations are not supported in atomic mode");
  P.n_extra = static_cast<int>(extra_ptrs.size());
  for (int e = 0; e < P.n_extra; ++e) P.C_extra[e] = reinterpret_cast<float*>(extra_ptrs[e]);
  plan.problems.push_back(P);
  std::vector<at::Tensor> keep = a_segs;
  keep.insert(keep.end(), b_segs.begin(), b_segs.end());
  if (C.has_value()) keep.push_back(*C);
  if (out_hi.has_value()) keep.push_back(*out_hi);
  if (out_lo.has_value()) keep.push_back(*out_lo);
  plan.keep_alive.push_back(std::move(keep));
}

void gemm_plan_finalize(int64_t id) {
  auto it = g_plans.find(id);
  TORCH_CHECK(it != g_plans.end() && !it->second.finalized, "unknown or finalized plan");
  GemmPlan& plan = it->second;
  TORCH_CHECK(!plan.problems.empty(), "empty plan");
  c10::cuda::CUDAGuard guard(plan.dev);
  DeviceState& st = device_state(plan.dev);
  // scratch for split-K problems (private to the plan)
  size_t scratch_floats = 0;
  for (auto& P : plan.problems)
    if (P.nsplit > 1 && !(P.flags & GF_ATOMIC))
      scratch_floats += static_cast<size_t>(P.ntiles) * P.nsplit * G_BM * G_BN;
  auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, plan.dev);
  if (scratch_floats > 0) plan.scratch = at::empty({static_cast<int64_t>(scratch_floats)}, f32);
  size_t off = 0;
  struct Item { int problem, tm, tn, split; long long cost; };
  std::vector<Item> items, ritems;
  for (size_t pi = 0; pi < plan.problems.size(); ++pi) {
    GemmProblem& P = plan.problems[pi];
    P.status = st.status.data_ptr<int>();
    const bool split = P.nsplit > 1 && !(P.flags & GF_ATOMIC);
    if (split) {
      P.ws = plan.scratch.data_ptr<float>() + off;
      off += static_cast<size_t>(P.ntiles) * P.nsplit * G_BM * G_BN;
    }
    const long long cost = static_cast<long long>(P.nseg) * ((P.K + G_BK - 1) / G_BK) / P.nsplit + 2;
    for (int tm = 0; tm < P.tiles_m; ++tm)
      for (int tn = 0; tn < ((P.flags & GF_SYM) ? tm + 1 : P.tiles_n); ++tn) {
        for (int s = 0; s < P.nsplit; ++s) items.push_back({static_cast<int>(pi), tm, tn, s, cost});
        if (split) ritems.push_back({static_cast<int>(pi), tm, tn, 0, 0});
      }
  }
  // longest tiles first: the tail of the launch is then made of short tiles
  std::stable_sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.cost > b.cost; });
  auto upload_work = [&](const std::vector<Item>& v) {
    std::vector<int> flat;
    flat.reserve(v.size() * 4);
    for (auto& w : v) {
      flat.push_back(w.problem);
      flat.push_back(w.tm);
      flat.push_back(w.tn);
      flat.push_back(w.split);
    }
    at::Tensor host = at::from_blob(flat.data(), {static_cast<int64_t>(flat.size())},
                                    at::TensorOptions().dtype(at::kInt)).clone();
    return host.to(at::Device(at::kCUDA, plan.dev));
  };
  plan.n_work = static_cast<int>(items.size());
  plan.n_rwork = static_cast<int>(ritems.size());
  plan.d_work = upload_work(items);
  if (plan.n_rwork > 0) plan.d_rwork = upload_work(ritems);
  at::Tensor host = at::from_blob(plan.problems.data(),
                                  {static_cast<int64_t>(plan.problems.size() * sizeof(GemmProblem))},
                                  at::TensorOptions().dtype(at::kByte)).clone();
  plan.d_problems = host.to(at::Device(at::kCUDA, plan.dev));
  TORCH_CHECK((reinterpret_cast<uintptr_t>(plan.d_problems.data_ptr()) & 63) == 0,
              "problem table is not 64-byte aligned");
  plan.finalized = true;
}

void gemm_plan_run(int64_t id) {
  auto it = g_plans.find(id);
  TORCH_CHECK(it != g_plans.end() && it->second.finalized, "unknown or unfinalized plan");
  GemmPlan& plan = it->second;
  c10::cuda::CUDAGuard guard(plan.dev);
  auto stream = at::cuda::getCurrentCUDAStream(plan.dev).stream();
  if (!g_attr_set) {
    B200_CUDA_CHECK(cudaFuncSetAttribute(umma_gemm_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, G_SMEM_BYTES));
    g_attr_set = true;
  }
  const GemmProblem* probs = reinterpret_cast<const GemmProblem*>(plan.d_problems.data_ptr());
  umma_gemm_kernel<<<plan.n_work, G_THREADS, G_SMEM_BYTES, stream>>>(
      plan.problems[0], probs, reinterpret_cast<const GemmWork*>(plan.d_work.data_ptr<int>()));
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
  if (plan.n_rwork > 0) {
    splitk_reduce_kernel<<<dim3(plan.n_rwork, 16, 1), 256, 0, stream>>>(
        plan.problems[0], probs, reinterpret_cast<const GemmWork*>(plan.d_rwork.data_ptr<int>()));
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
}

// Reads and clears the device status word (synchronises the current stream).
int64_t read_status(int64_t dev) {
  c10::cuda::CUDAGuard guard(static_cast<int>(dev));
  DeviceState& st = device_state(static_cast<int>(dev));
  int v = st.status.item<int>();
  if (v != 0) st.status.zero_();
  return v;
}

int64_t launch_count() { return static_cast<int64_t>(launch_counter().load()); }

void reserve_scratch(int64_t dev, int64_t nfloats) {
  c10::cuda::CUDAGuard guard(static_cast<int>(dev));
  ensure_scratch(static_cast<int>(dev), static_cast<size_t>(nfloats));
}

}  // namespace b200
