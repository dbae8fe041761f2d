// Host launcher for the persistent tcgen05 TN-GEMM / SYRK kernel (see umma_gemm2.cuh).
#include "gemm2_host.h"

#include <algorithm>
#include <unordered_map>

namespace b200 {

namespace {

// Split-K partials of single launches go through one scratch buffer per device, used as a ring.
// Launches on one stream reuse it in order; a launch on another stream first waits for the
// stream that used the ring last, so two streams never overlap on it.
struct Ring {
  size_t off = 0;
  cudaStream_t last = nullptr;
  bool used = false;
  cudaEvent_t ev = nullptr;
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

constexpr int kDefaultTileMode = 3;
bool g_batch_open = false;   // a deferred batch is recording (see gemm_batch_begin)
// 0: 128-wide tiles only, 1: 256-wide tiles for large outputs, 2: 256-wide wherever legal,
// 3: CTA-pair tiles (256 x 256, cta_group::2) for large products, 128-wide otherwise, 4: CTA pairs for every product
int g_wide_mode = kDefaultTileMode;

bool stream_is_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    cudaGetLastError();
    return true;
  }
  return st != cudaStreamCaptureStatusNone;
}

int tile_count(int tiles_m, int tiles_n, bool sym, int bn) {
  if (!sym) return tiles_m * tiles_n;
  int n = 0;
  for (int tm = 0; tm < tiles_m; ++tm) n += (tm * G2_BM) / bn + 1;
  return n;
}

}  // namespace

int g2_sm_count(int dev) {
  static int cached[64] = {0};
  if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
  const int n = at::cuda::getDeviceProperties(dev)->multiProcessorCount;
  if (dev >= 0 && dev < 64) cached[dev] = n;
  return n;
}

void g2_encode_operand(CUtensorMap* tm, const void* base, int64_t mn, int64_t k, int64_t ld,
                       bool kmajor, int box_mn) {
  if (kmajor)
    encode_tmap_bf16_2d(tm, base, k, mn, ld, 64, box_mn);
  else
    encode_tmap_bf16_2d(tm, base, mn, k, ld, 64, G2_BK);
}

void g2_launch_list(const GemmProblem2* d_probs, const GemmWork2* d_work, int n_work, G2Flavour flavour,
                    int dev, cudaStream_t stream) {
  if (n_work <= 0) return;
  GemmProblem2 dummy;
  std::memset(&dummy, 0, sizeof(dummy));
  const int n_sms = g2_sm_count(dev);
  if (flavour == G2_WIDE)
    g2_run_wide(dummy, d_probs, d_work, n_work, n_sms, stream);
  else if (flavour == G2_SPLIT3)
    g2_run_split3(dummy, d_probs, d_work, n_work, n_sms, stream);
  else if (flavour == G2_X3WIDE)
    g2_run_x3wide(dummy, d_probs, d_work, n_work, n_sms, stream);
  else
    g2_run_plain(dummy, d_probs, d_work, n_work, n_sms, stream);
}

void g2_launch_reduce_list(const GemmProblem2* d_probs, const GemmWork2* d_work, int n_work, bool wide,
                           cudaStream_t stream) {
  if (n_work <= 0) return;
  GemmProblem2 dummy;
  std::memset(&dummy, 0, sizeof(dummy));
  if (wide)
    splitk_reduce2_kernel<256><<<dim3(n_work, 32, 1), 256, 0, stream>>>(dummy, d_probs, d_work, nullptr, 0);
  else
    splitk_reduce2_kernel<128><<<dim3(n_work, 16, 1), 256, 0, stream>>>(dummy, d_probs, d_work, nullptr, 0);
  B200_CUDA_CHECK(cudaGetLastError());
  count_launch();
}

// Fills the scalar fields of a problem and encodes its tensor maps.
void gemm_fill_problem(GemmProblem2& P, const std::vector<at::Tensor>& a_segs,
                       const std::vector<at::Tensor>& b_segs, bool a_kmajor, bool b_kmajor,
                       const c10::optional<at::Tensor>& C, double alpha, double beta, bool sym,
                       const c10::optional<at::Tensor>& out_hi, const c10::optional<at::Tensor>& out_mid,
                       const c10::optional<at::Tensor>& out_lo, int64_t nsplit_req, bool split3, int n_sms,
                       bool allow_no_output = false, bool x3wide = false) {
  const int nseg = static_cast<int>(a_segs.size());
  TORCH_CHECK(nseg >= 1 && nseg <= G2_MAX_SEG && b_segs.size() == a_segs.size(),
              "between 1 and 6 operand segments are supported");
  TORCH_CHECK(!split3 || nseg == 3, "a split3 product takes the (hi, mid, lo) parts of both operands");
  TORCH_CHECK(!x3wide || (nseg == 2 && !split3), "an x3wide product takes the (hi, lo) parts of both operands");
  std::memset(&P, 0, sizeof(P));
  const at::Tensor& a0 = a_segs[0];
  const at::Tensor& b0 = b_segs[0];
  const int64_t M = a_kmajor ? a0.size(0) : a0.size(1);
  const int64_t K = a_kmajor ? a0.size(1) : a0.size(0);
  const int64_t N = b_kmajor ? b0.size(0) : b0.size(1);
  const int64_t Kb = b_kmajor ? b0.size(1) : b0.size(0);
  TORCH_CHECK(K == Kb, "contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(M > 0 && N > 0 && M < (1 << 30) && N < (1 << 30) && K < (1ll << 31) - 64, "matrix sizes out of range");
  if (sym) TORCH_CHECK(M == N, "symmetric mode needs a square output");
  const bool wide = x3wide || (!split3 && (g_wide_mode == 2 || (g_wide_mode == 1 && N >= 1024 && M >= 1024)));
  // CTA pairs pay from outputs of 2048 x 2048 and about 2e10 multiply-adds on (measured: 20 % faster than
  // 128-wide tiles at 4096 x 4096 x 8192, slower below 2048 x 2048 where a launch is a wave or less).  While a
  // batch is recording, a product leaves the batch for a pair launch of its own only from 1e11 multiply-adds
  // on: smaller ones fill the GPU better together with the rest of the batch.
  const double macs = static_cast<double>(M) * static_cast<double>(N) * static_cast<double>(K);
  const bool pair = !wide && !split3 &&
                    (g_wide_mode == 4 || (g_wide_mode == 3 && N >= 2048 && M >= 2048 && macs >= (g_batch_open ? 1e11 : 2e10)));
  const int bn = wide ? 256 : 128;        // B rows of a tensor-map box
  const int bn_grid = pair ? 256 : bn;    // tile width of the grid and of the split-K scratch
  for (int s = 0; s < nseg; ++s) {
    check_operand(a_segs[s], "A");
    check_operand(b_segs[s], "B");
    TORCH_CHECK(a_segs[s].sizes() == a0.sizes() && b_segs[s].sizes() == b0.sizes(),
                "all segments must have the same shape");
    g2_encode_operand(&P.tmA[s], a_segs[s].data_ptr(), M, K, a_segs[s].stride(0), a_kmajor, G2_BM);
    g2_encode_operand(&P.tmB[s], b_segs[s].data_ptr(), N, K, b_segs[s].stride(0), b_kmajor, bn);
  }
  bool same_ab = sym && !wide && !pair && !split3 && !x3wide && a_kmajor == b_kmajor;
  for (int s = 0; s < nseg && same_ab; ++s)
    same_ab = a_segs[s].data_ptr() == b_segs[s].data_ptr() &&
              a_segs[s].stride(0) == b_segs[s].stride(0);

  P.M = static_cast<int>(M);
  P.N = static_cast<int>(N);
  P.K = static_cast<int>(K);
  P.nseg = nseg;
  P.alpha = static_cast<float>(alpha);
  P.beta = static_cast<float>(beta);
  P.flags = (sym ? G2F_SYM : 0) | (a_kmajor ? G2F_A_KMAJOR : 0) | (b_kmajor ? G2F_B_KMAJOR : 0) |
            (same_ab ? G2F_SAME_AB : 0) | (wide ? G2F_WIDE : 0) | (split3 ? G2F_SPLIT3 : 0) |
            (x3wide ? G2F_SPLIT2 : 0) | (pair ? G2F_PAIR : 0);
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
    auto same_layout = [&](const at::Tensor& t) {
      return t.sizes() == h.sizes() && t.strides() == h.strides() && t.scalar_type() == at::kBFloat16 && t.is_cuda();
    };
    if (out_lo.has_value()) {
      TORCH_CHECK(same_layout(*out_lo), "out_lo must match out_hi");
      P.out_lo = reinterpret_cast<__nv_bfloat16*>(out_lo->data_ptr());
    }
    if (out_mid.has_value()) {
      TORCH_CHECK(out_lo.has_value() && same_layout(*out_mid), "out_mid needs out_lo and must match out_hi");
      P.out_mid = reinterpret_cast<__nv_bfloat16*>(out_mid->data_ptr());
    }
    if (sym) TORCH_CHECK(h.size(1) >= M, "bf16 outputs of a symmetric product are written on both triangles");
  } else {
    TORCH_CHECK(!out_lo.has_value() && !out_mid.has_value(), "out_lo / out_mid need out_hi");
  }
  TORCH_CHECK(allow_no_output || P.C != nullptr || P.out_hi != nullptr, "no output given");

  P.tiles_m = (P.M + G2_BM - 1) / G2_BM;
  P.tiles_n = (P.N + bn_grid - 1) / bn_grid;
  P.ntiles = tile_count(P.tiles_m, P.tiles_n, sym, bn_grid);
  const int kb_total = (P.K + G2_BK - 1) / G2_BK;
  int nsplit = split3 ? 1 : static_cast<int>(nsplit_req);  // the chunked sum of a split3 product is not split
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

static bool needs_ws(const GemmProblem2& P) { return P.nsplit > 1 && !(P.flags & G2F_ATOMIC); }
static int tile_width(const GemmProblem2& P) { return (P.flags & (G2F_WIDE | G2F_PAIR)) ? 256 : 128; }

void gemm_attach_scratch(GemmProblem2& P, int dev, cudaStream_t stream) {
  DeviceState& st = device_state(dev);
  P.status = st.status.data_ptr<int>();
  const int slot = dev & 15;
  if (needs_ws(P)) {
    const size_t need = static_cast<size_t>(P.ntiles) * P.nsplit * G2_BM * tile_width(P);
    const size_t cap_min = need * 4;
    float* base = ensure_scratch(dev, cap_min);
    const size_t cap = static_cast<size_t>(device_state(dev).scratch.numel());
    Ring& sr = g_scratch_ring[slot];
    if (sr.used && sr.last != stream && !stream_is_capturing(stream) && !stream_is_capturing(sr.last)) {
      // another stream used the ring last: order this launch after that stream's work
      if (sr.ev == nullptr) B200_CUDA_CHECK(cudaEventCreateWithFlags(&sr.ev, cudaEventDisableTiming));
      B200_CUDA_CHECK(cudaEventRecord(sr.ev, sr.last));
      B200_CUDA_CHECK(cudaStreamWaitEvent(stream, sr.ev, 0));
    }
    sr.last = stream;
    sr.used = true;
    if (sr.off + need > cap) sr.off = 0;
    P.ws = base + sr.off;
    sr.off += need;
  }
}

void gemm_launch_single(const GemmProblem2& P, int dev, cudaStream_t stream) {
  const int n_work = P.ntiles * P.nsplit;
  const int n_sms = g2_sm_count(dev);
  const bool wide = (P.flags & (G2F_WIDE | G2F_PAIR)) != 0;   // layout of the split-K scratch
  if (P.flags & G2F_PAIR)
    g2_run_pair(P, g2_pair_tiles(P) * P.nsplit, n_sms, stream);
  else if (P.flags & G2F_SPLIT3)
    g2_run_split3(P, nullptr, nullptr, n_work, n_sms, stream);
  else if (P.flags & G2F_SPLIT2)
    g2_run_x3wide(P, nullptr, nullptr, n_work, n_sms, stream);
  else if (wide)
    g2_run_wide(P, nullptr, nullptr, n_work, n_sms, stream);
  else
    g2_run_plain(P, nullptr, nullptr, n_work, n_sms, stream);
  if (needs_ws(P)) {
    if (wide)
      splitk_reduce2_kernel<256><<<dim3(P.ntiles, 32, 1), 256, 0, stream>>>(P, nullptr, nullptr, nullptr, 0);
    else
      splitk_reduce2_kernel<128><<<dim3(P.ntiles, 16, 1), 256, 0, stream>>>(P, nullptr, nullptr, nullptr, 0);
    B200_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
}

// ---- deferred batches ------------------------------------------------------------------------------
// Between gemm_batch_begin() and gemm_batch_end() the plain single-problem entry points do not launch:
// they record their problem (and keep its operands alive).  gemm_batch_end() runs everything recorded
// as ONE persistent launch (plus one split-K reduction launch).  The statistics products of a K-FAC
// curvature pass - about a hundred products whose tile counts range from 1 to 666 - fill the GPU
// together instead of one after the other.  The problem table reaches the device through kernel
// parameters (a few launches of a copy kernel with a 28 KiB argument), not through a host-to-device
// copy: parameters are captured by value, so a CUDA graph that contains a batch replays without
// referring to host memory.
struct GemmBatch {
  bool active = false;
  int dev = 0;
  std::vector<GemmProblem2> problems;
  std::vector<int> nsplit_req;
  std::vector<at::Tensor> keep_alive;
};
static GemmBatch g_batch;

constexpr int kTableChunk = 28 * 1024;
struct TableChunk {
  unsigned char bytes[kTableChunk];
};

__global__ void table_write_kernel(const __grid_constant__ TableChunk chunk, unsigned char* dst, int nbytes) {
  const int n16 = nbytes >> 4;   // nbytes and dst are multiples of 16
  const uint4* src = reinterpret_cast<const uint4*>(chunk.bytes);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) reinterpret_cast<uint4*>(dst)[i] = src[i];
}

static void batch_flush(cudaStream_t stream) {
  GemmBatch& B = g_batch;
  if (B.problems.empty()) return;
  c10::cuda::CUDAGuard guard(B.dev);
  DeviceState& st = device_state(B.dev);
  const int n_sms = g2_sm_count(B.dev);
  // split-K per problem: the batch fills the machine, so a split only has to cut very long contractions
  // into pieces of comparable length
  size_t ws_floats = 0;
  for (size_t i = 0; i < B.problems.size(); ++i) {
    GemmProblem2& P = B.problems[i];
    const int kb_total = (P.K + G2_BK - 1) / G2_BK;
    int nsplit = B.nsplit_req[i];
    if (nsplit <= 0) nsplit = std::min(32, std::max(1, kb_total / 48));
    nsplit = std::max(1, std::min(nsplit, kb_total));
    P.nsplit = nsplit;
    P.status = st.status.data_ptr<int>();
    if (needs_ws(P)) ws_floats += static_cast<size_t>(P.ntiles) * P.nsplit * G2_BM * 128;
  }
  // expensive items first
  std::vector<int> order(B.problems.size());
  for (size_t i = 0; i < order.size(); ++i) order[i] = static_cast<int>(i);
  auto item_cost = [&](int i) {
    const GemmProblem2& P = B.problems[i];
    return static_cast<long long>(P.nseg) * ((P.K + G2_BK - 1) / G2_BK) / P.nsplit;
  };
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return item_cost(a) > item_cost(b); });
  at::Tensor scratch;
  if (ws_floats > 0)
    scratch = at::empty({static_cast<int64_t>(ws_floats)}, at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, B.dev));
  size_t ws_off = 0;
  for (size_t begin = 0; begin < order.size(); begin += G2_MAX_BATCH) {
    const int n = static_cast<int>(std::min<size_t>(G2_MAX_BATCH, order.size() - begin));
    // table: [problems][item prefix (n + 1)][reduction tile prefix (n + 1)], 16-byte granular
    const size_t probs_bytes = static_cast<size_t>(n) * sizeof(GemmProblem2);
    const size_t prefix_bytes = ((static_cast<size_t>(n) + 1) * sizeof(int) + 15) / 16 * 16;
    const size_t total = probs_bytes + 2 * prefix_bytes;
    std::vector<unsigned char> host(total, 0);
    GemmProblem2* hp = reinterpret_cast<GemmProblem2*>(host.data());
    int* prefix = reinterpret_cast<int*>(host.data() + probs_bytes);
    int* rprefix = reinterpret_cast<int*>(host.data() + probs_bytes + prefix_bytes);
    int items = 0, rtiles = 0;
    for (int j = 0; j < n; ++j) {
      GemmProblem2 P = B.problems[order[begin + j]];
      if (needs_ws(P)) {
        P.ws = scratch.data_ptr<float>() + ws_off;
        ws_off += static_cast<size_t>(P.ntiles) * P.nsplit * G2_BM * 128;
      }
      hp[j] = P;
      prefix[j] = items;
      rprefix[j] = rtiles;
      items += P.ntiles * P.nsplit;
      if (needs_ws(P)) rtiles += P.ntiles;
    }
    prefix[n] = items;
    rprefix[n] = rtiles;
    at::Tensor table = at::empty({static_cast<int64_t>(total)}, at::TensorOptions().dtype(at::kByte).device(at::kCUDA, B.dev));
    unsigned char* d = table.data_ptr<unsigned char>();
    TORCH_CHECK((reinterpret_cast<uintptr_t>(d) & 63) == 0, "problem table is not 64-byte aligned");
    for (size_t off = 0; off < total; off += kTableChunk) {
      TableChunk chunk;
      const int nbytes = static_cast<int>(std::min<size_t>(kTableChunk, total - off));
      std::memcpy(chunk.bytes, host.data() + off, nbytes);
      table_write_kernel<<<1, 256, 0, stream>>>(chunk, d + off, nbytes);
      B200_CUDA_CHECK(cudaGetLastError());
      count_launch();
    }
    GemmProblem2 dummy;
    std::memset(&dummy, 0, sizeof(dummy));
    const GemmProblem2* dp = reinterpret_cast<const GemmProblem2*>(d);
    g2_run_plain(dummy, dp, nullptr, items, n_sms, stream, reinterpret_cast<const int*>(d + probs_bytes), n);
    if (rtiles > 0) {
      splitk_reduce2_kernel<128><<<dim3(rtiles, 16, 1), 256, 0, stream>>>(
          dummy, dp, nullptr, reinterpret_cast<const int*>(d + probs_bytes + prefix_bytes), n);
      B200_CUDA_CHECK(cudaGetLastError());
      count_launch();
    }
  }
  B.problems.clear();
  B.nsplit_req.clear();
  B.keep_alive.clear();
}

// Records `P` in the open batch.  Returns false when no batch is open (the caller launches itself).
static bool batch_append(GemmProblem2& P, int dev, int64_t nsplit_req, cudaStream_t stream,
                         const std::vector<at::Tensor>& a_segs, const std::vector<at::Tensor>& b_segs,
                         const c10::optional<at::Tensor>& C) {
  GemmBatch& B = g_batch;
  if (!B.active || (P.flags & (G2F_WIDE | G2F_SPLIT3 | G2F_SPLIT2 | G2F_PAIR))) return false;
  if (!B.problems.empty() && B.dev != dev) batch_flush(stream);
  // two products into one output (a further backward pass adding to a factor) must not share a launch
  for (const GemmProblem2& Q : B.problems)
    if (Q.C != nullptr && Q.C == P.C) {
      batch_flush(stream);
      break;
    }
  B.dev = dev;
  B.problems.push_back(P);
  B.nsplit_req.push_back(static_cast<int>(nsplit_req));
  B.keep_alive.insert(B.keep_alive.end(), a_segs.begin(), a_segs.end());
  B.keep_alive.insert(B.keep_alive.end(), b_segs.begin(), b_segs.end());
  if (C.has_value()) B.keep_alive.push_back(*C);
  return true;
}

void gemm_batch_begin() {
  TORCH_CHECK(!g_batch.active, "a GEMM batch is already open");
  g_batch.active = true;
  g_batch_open = true;
}

// Launches what was recorded since gemm_batch_begin() on the current stream; returns the number of products.
int64_t gemm_batch_end() {
  TORCH_CHECK(g_batch.active, "no GEMM batch is open");
  g_batch.active = false;
  g_batch_open = false;
  const int64_t n = static_cast<int64_t>(g_batch.problems.size());
  if (n > 0) {
    c10::cuda::CUDAGuard guard(g_batch.dev);
    batch_flush(at::cuda::getCurrentCUDAStream(g_batch.dev).stream());
  }
  return n;
}

// Drops an open batch without launching it (error paths).
void gemm_batch_abort() {
  g_batch.active = false;
  g_batch_open = false;
  g_batch.problems.clear();
  g_batch.nsplit_req.clear();
  g_batch.keep_alive.clear();
}

// Python entry: C = alpha * A^T B (+ beta C), optionally symmetric, optionally bf16 split outputs.
// `split3`: the three segments are the (hi, mid, lo) parts of fp32 operands and the product is
// formed fp32-grade (six part products, one accumulation chunk per K block; see umma_gemm2.cuh).
// `x3wide`: the two segments are the (hi, lo) parts of both operands (bf16x3 on 128 x 256 tiles).
void umma_gemm(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
               bool b_kmajor, c10::optional<at::Tensor> C, double alpha, double beta, bool sym,
               c10::optional<at::Tensor> out_hi, c10::optional<at::Tensor> out_lo,
               int64_t nsplit, c10::optional<at::Tensor> out_mid, bool split3, bool x3wide) {
  TORCH_CHECK(!a_segs.empty(), "no operands");
  const int dev = a_segs[0].get_device();
  c10::cuda::CUDAGuard guard(dev);
  GemmProblem2 P;
  gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, C, alpha, beta, sym, out_hi, out_mid, out_lo,
                    nsplit, split3, g2_sm_count(dev), false, x3wide);
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (out_hi.has_value() || !batch_append(P, dev, nsplit, stream, a_segs, b_segs, C)) {
    gemm_attach_scratch(P, dev, stream);
    gemm_launch_single(P, dev, stream);
  }
}

// Implicit-im2col SYRK: C = alpha * M^T M (+ beta * C) with M the patch matrix [n * oh * ow, kh * kw * c] of a
// stride-1, dilation-1 convolution input, columns ordered (kh, kw, c) - the input-side Kronecker factor of a
// convolution (asdl/operations/conv.py:80-88 builds M with unfold) without materialising M.
//   x: bf16 [n, c, h, w] in channels_last memory format (NHWC in memory), c a multiple of 64, kh * kw <= 12.
// The producer warp gathers every operand tile with 4-D TMA boxes of x (see G2F_CONV in umma_gemm2.cuh); the
// zero padding of the convolution and the output pixels past the image are TMA's out-of-bounds fill.
// With `dst_ptr` != 0 the result goes to that raw device address with pitch `ldc` instead of `C` (a symmetric-memory
// region); `mode` 3 stores the lower-triangular tiles only, 2 adds them with reductions (as in umma_gemm_to_ptr).
void umma_syrk_conv(at::Tensor x, c10::optional<at::Tensor> C_opt, int64_t kh, int64_t kw, int64_t ph, int64_t pw,
                    double alpha, double beta, int64_t nsplit_req, int64_t dst_ptr, int64_t ldc, int64_t mode) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 4 &&
                  x.is_contiguous(at::MemoryFormat::ChannelsLast),
              "x must be a 4-d channels_last bf16 CUDA tensor");
  const int64_t n = x.size(0), c = x.size(1), h = x.size(2), w = x.size(3);
  TORCH_CHECK(c % 64 == 0 && kh >= 1 && kw >= 1 && kh * kw <= 2 * G2_MAX_SEG && ph >= 0 && pw >= 0 && ph < kh && pw < kw,
              "implicit im2col needs a channel count that is a multiple of 64, at most 12 filter taps and padding below the filter size");
  const int64_t oh = h + 2 * ph - kh + 1, ow = w + 2 * pw - kw + 1;
  TORCH_CHECK(oh > ph && ow > pw && n >= 1, "the output must be larger than the padding");
  TORCH_CHECK((reinterpret_cast<uintptr_t>(x.data_ptr()) & 15) == 0, "x must be 16-byte aligned");
  const int64_t ncol = kh * kw * c;
  TORCH_CHECK((dst_ptr != 0) != C_opt.has_value(), "give either C or a destination address");
  float* c_ptr = nullptr;
  int64_t c_ld = 0;
  if (C_opt.has_value()) {
    const at::Tensor& C = *C_opt;
    TORCH_CHECK(C.is_cuda() && C.scalar_type() == at::kFloat && C.dim() == 2 && C.stride(1) == 1 && C.size(0) == ncol &&
                    C.size(1) == ncol,
                "C must be a [kh kw c, kh kw c] fp32 CUDA matrix with unit column stride");
    TORCH_CHECK(mode == 0, "lower-triangle modes write to a destination address");
    c_ptr = C.data_ptr<float>();
    c_ld = C.stride(0);
  } else {
    TORCH_CHECK(beta == 0.0 && (mode == 2 || mode == 3) && ldc >= ncol, "a destination address takes mode 2 or 3, beta 0 and ldc >= columns");
    c_ptr = reinterpret_cast<float*>(dst_ptr);
    c_ld = ldc;
  }
  TORCH_CHECK((reinterpret_cast<uintptr_t>(c_ptr) & 15) == 0 || (c_ld & 3) != 0,
              "the output must be 16-byte aligned when its row pitch is a multiple of four elements");
  const int dev = x.get_device();
  c10::cuda::CUDAGuard guard(dev);
  GemmProblem2 P;
  std::memset(&P, 0, sizeof(P));
  // pixel block of a K step: bw x bh output pixels of bi images, bw * bh * bi = 64, least overhang (ties: widest rows)
  int bw = 8, bh = 8, bi = 1;
  {
    long long best = -1;
    for (int a = 6; a >= 0; --a)
      for (int b = 6 - a; b >= 0; --b) {
        const int cw = 1 << a, ch = 1 << b, ci = 1 << (6 - a - b);
        const long long vol = ((ow + cw - 1) / cw) * cw * ((oh + ch - 1) / ch) * ch * ((n + ci - 1) / ci) * ci;
        if (best < 0 || vol < best) {
          best = vol;
          bw = cw;
          bh = ch;
          bi = ci;
        }
      }
  }
  const int th = static_cast<int>((oh + bh - 1) / bh), tw = static_cast<int>((ow + bw - 1) / bw);
  const int ti = static_cast<int>((n + bi - 1) / bi);
  TORCH_CHECK(static_cast<long long>(ti) * th * tw < (1ll << 24), "too many pixel blocks");
  for (int q = 0; q < kh * kw; ++q) {
    const int64_t khh = q / kw, kww = q % kw;
    // extents of tap q: the last valid output pixel (oh - 1, ow - 1) reads input (oh - 1 + khh - ph, ow - 1 + kww - pw)
    const cuuint64_t wq = static_cast<cuuint64_t>(std::min<int64_t>(w, ow + kww - pw));
    const cuuint64_t hq = static_cast<cuuint64_t>(std::min<int64_t>(h, oh + khh - ph));
    cuuint64_t dims[4] = {static_cast<cuuint64_t>(c), wq, hq, static_cast<cuuint64_t>(n)};
    cuuint64_t strides[3] = {static_cast<cuuint64_t>(c) * 2, static_cast<cuuint64_t>(w * c) * 2,
                             static_cast<cuuint64_t>(h * w * c) * 2};
    cuuint32_t box[4] = {64, static_cast<cuuint32_t>(bw), static_cast<cuuint32_t>(bh), static_cast<cuuint32_t>(bi)};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUtensorMap* tm = q < G2_MAX_SEG ? &P.tmA[q] : &P.tmB[q - G2_MAX_SEG];
    CUresult r = get_encode_tiled()(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, x.data_ptr(), dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TORCH_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (4-d) failed with code ", static_cast<int>(r));
  }
  P.M = P.N = static_cast<int>(ncol);
  P.K = ti * th * tw * G2_BK;   // 64 output pixels per K block
  P.nseg = 1;
  P.alpha = static_cast<float>(alpha);
  P.beta = static_cast<float>(beta);
  P.flags = G2F_SYM | G2F_SAME_AB | G2F_CONV | (mode == 2 ? G2F_ATOMIC : 0) | (mode >= 2 ? G2F_LOWER : 0);
  P.C = c_ptr;
  P.Cin = P.C;
  P.ldc = static_cast<int>(c_ld);
  P.conv_c = static_cast<int>(c);
  P.conv_kw = static_cast<int>(kw);
  P.conv_taps = static_cast<int>(kh * kw);
  P.conv_ph = static_cast<int>(ph);
  P.conv_pw = static_cast<int>(pw);
  P.conv_th = th;
  P.conv_tw = tw;
  P.conv_box = bw | (bh << 8) | (bi << 16);
  P.tiles_m = (P.M + G2_BM - 1) / G2_BM;
  P.tiles_n = (P.N + 127) / 128;
  P.ntiles = tile_count(P.tiles_m, P.tiles_n, true, 128);
  const int kb_total = P.K / G2_BK;
  int nsplit = static_cast<int>(nsplit_req);
  if (nsplit <= 0) {
    nsplit = (2 * g2_sm_count(dev)) / std::max(P.ntiles, 1);
    nsplit = std::min(std::min(nsplit, kb_total / 8), 32);
  }
  P.nsplit = std::max(1, std::min(nsplit, kb_total));
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (!batch_append(P, dev, nsplit_req, stream, {x}, {}, C_opt)) {
    gemm_attach_scratch(P, dev, stream);
    gemm_launch_single(P, dev, stream);
  }
}

// Variant whose fp32 result goes to raw device addresses - typically symmetric-memory buffers of
// this or another GPU.  `dst_ptr` receives the result (accumulated with reductions when `atomic`),
// `extra_ptrs` receive plain copies of it (non-atomic mode only).  All destinations use `ldc`.
void umma_gemm_to_ptr(std::vector<at::Tensor> a_segs, std::vector<at::Tensor> b_segs, bool a_kmajor,
                      bool b_kmajor, int64_t dst_ptr, int64_t ldc, double alpha, bool sym, int64_t atomic,
                      std::vector<int64_t> extra_ptrs, int64_t nsplit, bool mcast) {
  TORCH_CHECK(!a_segs.empty(), "no operands");
  TORCH_CHECK(dst_ptr != 0 && (dst_ptr & 15) == 0, "destination must be a 16-byte aligned device address");
  TORCH_CHECK(static_cast<int>(extra_ptrs.size()) <= G2_MAX_EXTRA, "too many extra destinations");
  TORCH_CHECK(!((atomic == 1 || atomic == 2) && !extra_ptrs.empty()),
              "extra destinations are not supported in atomic mode");
  const int dev = a_segs[0].get_device();
  c10::cuda::CUDAGuard guard(dev);
  GemmProblem2 P;
  gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, c10::nullopt, alpha, 0.0, sym,
                    c10::nullopt, c10::nullopt, c10::nullopt, nsplit, false, g2_sm_count(dev),
                    /*allow_no_output=*/true);
  P.C = reinterpret_cast<float*>(dst_ptr);
  P.Cin = P.C;
  P.ldc = static_cast<int>(ldc);
  TORCH_CHECK(P.ldc >= P.N, "ldc is smaller than the number of columns");
  if (atomic == 1 || atomic == 2) P.flags |= G2F_ATOMIC;
  if (atomic == 2 || atomic == 3) {
    TORCH_CHECK(sym, "lower-triangle output needs the symmetric mode");
    P.flags |= G2F_LOWER;
  }
  P.n_extra = static_cast<int>(extra_ptrs.size());
  for (int e = 0; e < P.n_extra; ++e) {
    TORCH_CHECK((extra_ptrs[e] & 15) == 0, "destinations must be 16-byte aligned");
    P.C_extra[e] = reinterpret_cast<float*>(extra_ptrs[e]);
  }
  if (mcast) {
    TORCH_CHECK(!sym && atomic == 0, "multicast destinations take the plain result of a non-symmetric product");
    P.flags |= G2F_MCAST;
  }
  auto stream = at::cuda::getCurrentCUDAStream(dev).stream();
  if (!batch_append(P, dev, nsplit, stream, a_segs, b_segs, c10::nullopt)) {
    gemm_attach_scratch(P, dev, stream);
    gemm_launch_single(P, dev, stream);
  }
}

// ---- grouped execution ---------------------------------------------------------------------------
// A plan is a fixed list of GEMM problems whose operand addresses do not change (persistent
// buffers).  Its problem table and tile list live in device memory, so running the plan is two
// launches at most (all tiles of all problems on persistent CTAs, then the split-K reductions)
// with no host-side descriptor work - which also makes it replayable from a CUDA graph.
struct GemmPlan {
  std::vector<GemmProblem2> problems;
  std::vector<std::vector<at::Tensor>> keep_alive;  // operands / outputs referenced by raw pointer
  at::Tensor d_problems, d_work, d_rwork, scratch;
  int n_work = 0, n_rwork = 0, dev = 0;
  int split3 = -1;  // -1: no problem yet, 0: plain products, 1: split3, 2: x3wide (never mixed)
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
                   int64_t nsplit, c10::optional<at::Tensor> out_mid, bool split3, bool x3wide, bool mcast) {
  auto it = g_plans.find(id);
  TORCH_CHECK(it != g_plans.end() && !it->second.finalized, "unknown or finalized plan");
  GemmPlan& plan = it->second;
  TORCH_CHECK(!a_segs.empty(), "no operands");
  plan.dev = a_segs[0].get_device();
  const int kind = split3 ? 1 : (x3wide ? 2 : 0);
  TORCH_CHECK(plan.split3 < 0 || plan.split3 == kind, "a plan holds products of one kind (plain, split3 or x3wide)");
  TORCH_CHECK(!(x3wide && sym), "symmetric products are not supported in x3wide plans");
  plan.split3 = kind;
  c10::cuda::CUDAGuard guard(plan.dev);
  GemmProblem2 P;
  const int saved_mode = g_wide_mode;
  g_wide_mode = 0;  // the tiles of a plan share one kernel instantiation: 128-wide
  try {
    gemm_fill_problem(P, a_segs, b_segs, a_kmajor, b_kmajor, C, alpha, beta, sym, out_hi, out_mid, out_lo,
                      nsplit <= 0 ? 1 : nsplit, split3, g2_sm_count(plan.dev), /*allow_no_output=*/dst_ptr != 0 || !extra_ptrs.empty(), x3wide);
  } catch (...) {
    g_wide_mode = saved_mode;
    throw;
  }
  g_wide_mode = saved_mode;
  if (dst_ptr != 0) {
    TORCH_CHECK((dst_ptr & 15) == 0, "destination must be 16-byte aligned");
    P.C = reinterpret_cast<float*>(dst_ptr);
    P.Cin = P.C;
  }
  if (dst_ptr != 0 || !extra_ptrs.empty()) {
    P.ldc = static_cast<int>(ldc);
    TORCH_CHECK(P.ldc >= P.N, "ldc is smaller than the number of columns");
  }
  if (atomic) P.flags |= G2F_ATOMIC;
  TORCH_CHECK(static_cast<int>(extra_ptrs.size()) <= G2_MAX_EXTRA, "too many extra destinations");
  TORCH_CHECK(!(atomic && !extra_ptrs.empty()), "extra destinations are not supported in atomic mode");
  P.n_extra = static_cast<int>(extra_ptrs.size());
  for (int e = 0; e < P.n_extra; ++e) P.C_extra[e] = reinterpret_cast<float*>(extra_ptrs[e]);
  if (mcast) {
    TORCH_CHECK(!sym && !atomic, "multicast destinations take the plain result of a non-symmetric product");
    P.flags |= G2F_MCAST;
  }
  plan.problems.push_back(P);
  std::vector<at::Tensor> keep = a_segs;
  keep.insert(keep.end(), b_segs.begin(), b_segs.end());
  if (C.has_value()) keep.push_back(*C);
  if (out_hi.has_value()) keep.push_back(*out_hi);
  if (out_mid.has_value()) keep.push_back(*out_mid);
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
    if (needs_ws(P)) scratch_floats += static_cast<size_t>(P.ntiles) * P.nsplit * G2_BM * tile_width(P);
  auto f32 = at::TensorOptions().dtype(at::kFloat).device(at::kCUDA, plan.dev);
  if (scratch_floats > 0) plan.scratch = at::empty({static_cast<int64_t>(scratch_floats)}, f32);
  size_t off = 0;
  struct Item {
    GemmWork2 w;
    long long cost;
  };
  std::vector<Item> items, ritems;
  for (size_t pi = 0; pi < plan.problems.size(); ++pi) {
    GemmProblem2& P = plan.problems[pi];
    P.status = st.status.data_ptr<int>();
    const bool split = needs_ws(P);
    if (split) {
      P.ws = plan.scratch.data_ptr<float>() + off;
      off += static_cast<size_t>(P.ntiles) * P.nsplit * G2_BM * tile_width(P);
    }
    const int kb_total = (P.K + G2_BK - 1) / G2_BK;
    const int bn = tile_width(P);
    int tile = 0;
    for (int tm = 0; tm < P.tiles_m; ++tm)
      for (int tn = 0; tn < ((P.flags & G2F_SYM) ? tm + 1 : P.tiles_n); ++tn, ++tile) {
        for (int s = 0; s < P.nsplit; ++s) {
          const int kb0 = static_cast<int>((static_cast<long long>(s) * kb_total) / P.nsplit);
          const int kb1 = static_cast<int>((static_cast<long long>(s + 1) * kb_total) / P.nsplit);
          GemmWork2 w;
          std::memset(&w, 0, sizeof(w));
          w.problem = static_cast<int>(pi);
          w.a_mn = w.c_row = tm * G2_BM;
          w.b_mn = w.c_col = tn * bn;
          w.a_k0 = w.b_k0 = kb0 * G2_BK;
          w.nkb = kb1 - kb0;
          w.tile_id = tile;
          w.split = s;
          items.push_back({w, static_cast<long long>((P.flags & G2F_SPLIT3) ? 6 : ((P.flags & G2F_SPLIT2) ? 6 : P.nseg)) *
                                  w.nkb + 2});
          if (split && s == 0) ritems.push_back({w, 0});
        }
      }
  }
  // longest tiles first: with CTAs taking items round-robin the tail is made of short tiles
  std::stable_sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.cost > b.cost; });
  auto upload_work = [&](const std::vector<Item>& v) {
    std::vector<GemmWork2> flat;
    flat.reserve(v.size());
    for (auto& w : v) flat.push_back(w.w);
    at::Tensor host = at::from_blob(flat.data(), {static_cast<int64_t>(flat.size() * sizeof(GemmWork2))},
                                    at::TensorOptions().dtype(at::kByte)).clone();
    return host.to(at::Device(at::kCUDA, plan.dev));
  };
  plan.n_work = static_cast<int>(items.size());
  plan.n_rwork = static_cast<int>(ritems.size());
  plan.d_work = upload_work(items);
  if (plan.n_rwork > 0) plan.d_rwork = upload_work(ritems);
  at::Tensor host = at::from_blob(plan.problems.data(),
                                  {static_cast<int64_t>(plan.problems.size() * sizeof(GemmProblem2))},
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
  const GemmProblem2* probs = reinterpret_cast<const GemmProblem2*>(plan.d_problems.data_ptr());
  g2_launch_list(probs, reinterpret_cast<const GemmWork2*>(plan.d_work.data_ptr()), plan.n_work,
                 plan.split3 == 1 ? G2_SPLIT3 : (plan.split3 == 2 ? G2_X3WIDE : G2_PLAIN), plan.dev, stream);
  if (plan.n_rwork > 0)
    g2_launch_reduce_list(probs, reinterpret_cast<const GemmWork2*>(plan.d_rwork.data_ptr()), plan.n_rwork,
                          plan.split3 == 2, stream);
}

// Tile policy of the single-problem entry points.  0: 128-wide tiles only; 1: 256-wide tiles for outputs of
// at least 1024 x 1024; 2: 256-wide wherever legal; 3 (the default): CTA-pair tiles (256 x 256 over two SMs,
// cta_group::2) for large products and 128-wide tiles otherwise; 4: CTA pairs for every product; -1: the default.
void set_gemm_wide(int64_t mode) {
  TORCH_CHECK(mode >= -1 && mode <= 4, "mode must be -1 (default), 0, 1, 2, 3 or 4");
  g_wide_mode = mode < 0 ? kDefaultTileMode : static_cast<int>(mode);
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
