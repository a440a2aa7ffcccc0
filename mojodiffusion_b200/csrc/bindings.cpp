// torch.ops.mdb200.* : thin host bindings that unpack tensors into the C launch structs of the kernels.
// No math happens here. Every kernel reports device-side failures (bounded waits that ran out) into one
// per-device status block that `mdb200::check_status` reads back.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "comm_api.h"
#include "gemm_api.h"
#include "kernels_api.h"

namespace {

using at::Tensor;
using c10::optional;

std::mutex g_mu;
std::atomic<long long> g_launches{0};
std::map<int, Tensor> g_status;

int* status_ptr(const Tensor& like) {
  std::lock_guard<std::mutex> lk(g_mu);
  const int dev = like.get_device();
  auto it = g_status.find(dev);
  if (it == g_status.end()) {
    Tensor t = at::zeros({4}, like.options().dtype(at::kInt));
    it = g_status.emplace(dev, t).first;
  }
  return it->second.data_ptr<int>();
}

void check_rc(int rc, const char* what) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  TORCH_CHECK(rc == 0, "mdb200 kernel launch failed in ", what, ": code ", rc,
              rc > 0 && rc < 1000 ? std::string(" (") + cudaGetErrorString(static_cast<cudaError_t>(rc)) + ")" : "");
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

const void* opt_ptr(const optional<Tensor>& t) { return t.has_value() && t->defined() ? t->data_ptr() : nullptr; }

// ------------------------------------------------------------------------------------------
// GEMM
// ------------------------------------------------------------------------------------------
Tensor gemm(std::vector<Tensor> As, std::vector<Tensor> Bs, const optional<Tensor>& bias,
            const optional<Tensor>& residual, const optional<Tensor>& gate, int64_t rows_per_group, int64_t act,
            int64_t pair_offset, int64_t act_on_second, const optional<Tensor>& out_opt, bool out_fp32, bool a_mn,
            bool b_mn, const optional<Tensor>& row_scale, const optional<Tensor>& col_scale, double alpha,
            bool accumulate, int64_t bn, const optional<Tensor>& prof, std::vector<int64_t> route_ptrs,
            std::vector<int64_t> route_cfg, std::vector<int64_t> gather_ptrs, std::vector<int64_t> gather_cfg,
            const optional<Tensor>& gather_dst, const optional<Tensor>& gather_ready, int64_t split_k) {
  TORCH_CHECK(!As.empty() && As.size() == Bs.size() && As.size() <= MDB_GEMM_MAX_SEG, "gemm: 1..3 K segments");
  const Tensor& A0 = As[0];
  TORCH_CHECK(A0.is_cuda(), "gemm: CUDA tensors only");
  c10::cuda::CUDAGuard guard(A0.device());
  const bool fp8 = A0.scalar_type() == at::kFloat8_e4m3fn;
  MdbGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.kind = fp8 ? 1 : 0;
  g.a_mn = a_mn;
  g.b_mn = b_mn;
  const int64_t M = a_mn ? A0.size(1) : A0.size(0);
  const int64_t Nrows = b_mn ? Bs[0].size(1) : Bs[0].size(0);
  const int64_t N = pair_offset > 0 ? pair_offset : Nrows;
  TORCH_CHECK(pair_offset <= 0 || Nrows == 2 * pair_offset, "gemm: paired mode wants B with 2*pair_offset rows");
  g.M = static_cast<int>(M);
  g.N = static_cast<int>(N);
  g.num_seg = static_cast<int>(As.size());
  const int align = fp8 ? 16 : 8;
  for (size_t s = 0; s < As.size(); ++s) {
    const Tensor& A = As[s];
    const Tensor& B = Bs[s];
    TORCH_CHECK(A.dim() == 2 && B.dim() == 2 && A.stride(1) == 1 && B.stride(1) == 1, "gemm: 2-D row-major operands");
    TORCH_CHECK(A.scalar_type() == A0.scalar_type() && B.scalar_type() == A0.scalar_type(), "gemm: dtype mismatch");
    TORCH_CHECK(fp8 || A.scalar_type() == at::kBFloat16, "gemm: bf16 or float8_e4m3fn operands");
    const int64_t K = a_mn ? A.size(0) : A.size(1);
    TORCH_CHECK((b_mn ? B.size(0) : B.size(1)) == K, "gemm: K mismatch in segment ", s);
    TORCH_CHECK((a_mn ? A.size(1) : A.size(0)) == M, "gemm: M mismatch in segment ", s);
    TORCH_CHECK((b_mn ? B.size(1) : B.size(0)) == Nrows, "gemm: N mismatch in segment ", s);
    TORCH_CHECK(A.stride(0) % align == 0 && B.stride(0) % align == 0, "gemm: leading dims must be 16-byte multiples");
    TORCH_CHECK(reinterpret_cast<uintptr_t>(A.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(B.data_ptr()) % 16 == 0,
                "gemm: operands must be 16-byte aligned");
    g.K[s] = K;
    g.A[s] = A.data_ptr();
    g.B[s] = B.data_ptr();
    g.lda[s] = A.stride(0);
    g.ldb[s] = B.stride(0);
  }
  Tensor out;
  if (!route_ptrs.empty()) {
    out = at::empty({0}, A0.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  } else if (out_opt.has_value() && out_opt->defined()) {
    out = *out_opt;
    TORCH_CHECK(out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1, "gemm: bad out shape");
    TORCH_CHECK(out.scalar_type() == (out_fp32 ? at::kFloat : at::kBFloat16), "gemm: out dtype");
  } else {
    out = at::empty({M, N}, A0.options().dtype(out_fp32 ? at::kFloat : at::kBFloat16));
  }
  TORCH_CHECK(!accumulate || out_fp32, "gemm: accumulate needs an fp32 output");
  g.out = out.data_ptr();
  g.ld_out = out.dim() == 2 ? static_cast<int>(out.stride(0)) : 0;
  g.out_fp32 = out_fp32;
  g.accumulate_out = accumulate;
  g.bn = static_cast<int>(bn);
  g.split_k = static_cast<int>(split_k);
  TORCH_CHECK(split_k <= 1 || (out_fp32 && out_opt.has_value()), "gemm: split-K adds into a caller-zeroed fp32 out");
  g.pair_offset = static_cast<int>(pair_offset > 0 ? pair_offset : 0);
  g.act = static_cast<int>(act);
  g.act_on_second = static_cast<int>(act_on_second);
  g.alpha = static_cast<float>(alpha);
  if (bias.has_value() && bias->defined()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == Nrows, "gemm: bias");
    g.bias = bias->data_ptr();
  }
  if (row_scale.has_value() && row_scale->defined()) {
    TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->numel() == M, "gemm: row_scale");
    g.row_scale = row_scale->data_ptr<float>();
  }
  if (col_scale.has_value() && col_scale->defined()) {
    TORCH_CHECK(col_scale->scalar_type() == at::kFloat && col_scale->numel() == Nrows, "gemm: col_scale");
    g.col_scale = col_scale->data_ptr<float>();
  }
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == M &&
                    residual->size(1) == N && residual->stride(1) == 1,
                "gemm: residual");
    g.residual = residual->data_ptr();
    g.ld_res = static_cast<int>(residual->stride(0));
  }
  if (gate.has_value() && gate->defined()) {
    TORCH_CHECK(gate->scalar_type() == at::kBFloat16 && gate->dim() == 2 && gate->size(1) == N && gate->stride(1) == 1,
                "gemm: gate must be [groups, N] bf16");
    TORCH_CHECK(rows_per_group > 0 && gate->size(0) * rows_per_group >= M, "gemm: gate groups do not cover M");
    g.gate = gate->data_ptr();
    g.gate_stride = static_cast<int>(gate->stride(0));
  }
  g.rows_per_group = static_cast<int>(rows_per_group > 0 ? rows_per_group : 1);
  g.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  g.status = status_ptr(A0);
  if (prof.has_value() && prof->defined()) {
    TORCH_CHECK(prof->scalar_type() == at::kLong && prof->numel() >= 8 * g.num_sms, "gemm: prof [sms, 8] int64");
    g.prof = reinterpret_cast<long long*>(prof->data_ptr());
    const int64_t extra = prof->numel() - 8 * g.num_sms;
    if (extra >= 6 * 64) {                       // room behind the counters: per-K-block time line of CTAs 0 and 1
      g.trace = g.prof + 8 * g.num_sms;
      g.trace_len = static_cast<int>(extra / 6);
    }
  }
  if (!gather_ptrs.empty()) {
    // gather_cfg = {rank, operand (0 A / 1 B), chunk_rows, chunk_bytes}
    TORCH_CHECK(gather_ptrs.size() <= MDB_GEMM_MAX_PEERS && gather_cfg.size() == 4 && gather_dst.has_value() &&
                    gather_ready.has_value() && gather_ready->scalar_type() == at::kInt && gather_ready->numel() >= 8,
                "gemm: gather arguments");
    for (size_t i = 0; i < gather_ptrs.size(); ++i) g.gather_src[i] = reinterpret_cast<const void*>(gather_ptrs[i]);
    g.gather_world = (int)gather_ptrs.size();
    g.gather_rank = (int)gather_cfg[0];
    g.gather_operand = (int)gather_cfg[1];
    g.gather_chunk_rows = (int)gather_cfg[2];
    g.gather_chunk_bytes = gather_cfg[3];
    g.gather_dst = gather_dst->data_ptr();
    g.gather_ready = gather_ready->data_ptr<int>();
  }
  g.reduce_src_rank = -1;
  if (!route_ptrs.empty() && route_cfg.size() == 3) {
    // staged reduce-scatter epilogue: route_cfg = {rows_per_owner, ld_out, this rank}; bf16 rows go to slot `rank` of
    // the owner's [world, rows_per_owner, ld_out] staging buffer
    TORCH_CHECK(!out_fp32, "gemm: the staged reduce-scatter epilogue stores bf16");
    for (size_t i = 0; i < route_ptrs.size(); ++i) g.route_out[i] = reinterpret_cast<void*>(route_ptrs[i]);
    g.reduce_rows_per_owner = (int)route_cfg[0];
    g.ld_out = (int)route_cfg[1];
    g.reduce_src_rank = (int)route_cfg[2];
  } else if (!route_ptrs.empty() && route_cfg.size() == 2) {
    // reduce-scatter epilogue: route_cfg = {rows_per_owner, ld_out}
    TORCH_CHECK(out_fp32, "gemm: reduce-scatter epilogue accumulates in fp32");
    for (size_t i = 0; i < route_ptrs.size(); ++i) g.route_out[i] = reinterpret_cast<void*>(route_ptrs[i]);
    g.reduce_rows_per_owner = (int)route_cfg[0];
    g.ld_out = (int)route_cfg[1];
  } else if (!route_ptrs.empty()) {
    // route_cfg = {owner_cols, part_cols, row_offset, rows_per_batch, batch_rows, ld_out[, split, row_offset_b]}
    TORCH_CHECK(route_ptrs.size() <= MDB_GEMM_MAX_PEERS && (route_cfg.size() == 6 || route_cfg.size() == 8), "gemm: route arguments");
    if (route_cfg.size() == 8) {
      g.route_split = (int)route_cfg[6];
      g.route_row_offset_b = (int)route_cfg[7];
    }
    for (size_t i = 0; i < route_ptrs.size(); ++i) g.route_out[i] = reinterpret_cast<void*>(route_ptrs[i]);
    g.route_owner_cols = (int)route_cfg[0];
    g.route_part_cols = (int)route_cfg[1];
    g.route_row_offset = (int)route_cfg[2];
    g.route_rows_per_batch = (int)route_cfg[3];
    g.route_batch_rows = (int)route_cfg[4];
    g.ld_out = (int)route_cfg[5];
    TORCH_CHECK((int64_t)route_ptrs.size() * g.route_owner_cols == g.route_part_cols && N % g.route_part_cols == 0,
                "gemm: route blocks do not tile the output columns");
  }
  check_rc(mdb_gemm_launch(&g, cur_stream()), "gemm");
  return out;
}

// x: NHWC bf16 [N, H, W, Cin]; w: [Cout, KH, KW, Cin] bf16; stride 1, "same"-style padding (pad_h, pad_w).
Tensor conv2d_nhwc(const Tensor& x, const Tensor& w, const optional<Tensor>& bias, int64_t pad_h, int64_t pad_w,
                   int64_t act, const optional<Tensor>& residual) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && w.dim() == 4 && x.is_contiguous() && w.is_contiguous(), "conv2d_nhwc: NHWC");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w.scalar_type() == at::kBFloat16, "conv2d_nhwc: bf16");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t N = x.size(0), H = x.size(1), W = x.size(2), Cin = x.size(3);
  const int64_t Cout = w.size(0), KH = w.size(1), KW = w.size(2);
  TORCH_CHECK(w.size(3) == Cin && Cin % 64 == 0 && Cout % 8 == 0, "conv2d_nhwc: Cin multiple of 64, Cout multiple of 8");
  TORCH_CHECK(2 * pad_h == KH - 1 && 2 * pad_w == KW - 1, "conv2d_nhwc: output size must equal input size");
  Tensor out = at::empty({N, H, W, Cout}, x.options());
  MdbGemmArgs g;
  memset(&g, 0, sizeof(g));
  g.M = (int)(N * H * W); g.N = (int)Cout; g.num_seg = 1;
  g.K[0] = KH * KW * Cin;
  g.A[0] = x.data_ptr(); g.B[0] = w.data_ptr();
  g.lda[0] = Cin; g.ldb[0] = KH * KW * Cin;
  g.alpha = 1.f; g.act = (int)act;
  g.out = out.data_ptr(); g.ld_out = (int)Cout;
  g.rows_per_group = 1;
  if (bias.has_value() && bias->defined()) g.bias = bias->data_ptr();
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_contiguous() && residual->numel() == out.numel(), "conv2d_nhwc: residual shape");
    g.residual = residual->data_ptr();
    g.ld_res = (int)Cout;
  }
  g.conv_taps = (int)(KH * KW); g.conv_kw = (int)KW; g.conv_pad_h = (int)pad_h; g.conv_pad_w = (int)pad_w;
  g.conv_n = (int)N; g.conv_h = (int)H; g.conv_w = (int)W; g.conv_cin = (int)Cin;
  g.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  g.status = status_ptr(x);
  check_rc(mdb_gemm_launch(&g, cur_stream()), "conv2d_nhwc");
  return out;
}

Tensor group_norm_nhwc(const Tensor& x, const optional<Tensor>& w, const optional<Tensor>& b, int64_t groups, double eps,
                       int64_t act) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "group_norm_nhwc");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  Tensor stats = at::empty({mdb_group_norm_scratch_floats((int)x.size(0), (int)(x.size(1) * x.size(2)), (int)x.size(3), (int)groups, -1)},
                           x.options().dtype(at::kFloat));
  check_rc(mdb_group_norm(x.data_ptr(), y.data_ptr(), stats.data_ptr<float>(), opt_ptr(w), opt_ptr(b), (int)x.size(0),
                          (int)(x.size(1) * x.size(2)), (int)x.size(3), (int)groups, (float)eps, (int)act, cur_stream()),
           "group_norm");
  return y;
}
// -> {dx, dw (fp32 [C] or empty), db}
std::tuple<Tensor, Tensor, Tensor> group_norm_nhwc_bwd(const Tensor& x, const Tensor& dy, const optional<Tensor>& w, const optional<Tensor>& b,
                                                       int64_t groups, double eps, int64_t act, bool need_wgrad) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "group_norm_nhwc_bwd: x");
  TORCH_CHECK(dy.is_cuda() && dy.is_contiguous() && dy.scalar_type() == at::kBFloat16 && dy.sizes() == x.sizes() && dy.device() == x.device(),
              "group_norm_nhwc_bwd: dy must match x");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t C = x.size(3);
  Tensor dx = at::empty_like(x);
  Tensor scratch = at::empty({mdb_group_norm_scratch_floats((int)x.size(0), (int)(x.size(1) * x.size(2)), (int)C, (int)groups, need_wgrad ? 1 : 0)},
                             x.options().dtype(at::kFloat));
  Tensor dw, db;
  if (need_wgrad) {
    dw = at::zeros({C}, x.options().dtype(at::kFloat));
    db = at::zeros({C}, x.options().dtype(at::kFloat));
  }
  float* st = scratch.data_ptr<float>();
  g_launches.fetch_add(3, std::memory_order_relaxed);
  check_rc(mdb_group_norm_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), st, opt_ptr(w), opt_ptr(b),
                              need_wgrad ? dw.data_ptr<float>() : nullptr, need_wgrad ? db.data_ptr<float>() : nullptr, (int)x.size(0),
                              (int)(x.size(1) * x.size(2)), (int)C, (int)groups, (float)eps, (int)act, cur_stream()),
           "group_norm_bwd");
  return {dx, need_wgrad ? dw : Tensor(), need_wgrad ? db : Tensor()};
}
Tensor image_filter(int64_t op, const Tensor& img, const std::vector<double>& params, const optional<Tensor>& aux) {
  TORCH_CHECK(img.is_cuda() && img.dim() == 3 && img.size(2) == 4 && img.is_contiguous() && img.scalar_type() == at::kFloat,
              "image_filter: fp32 contiguous [H, W, 4] expected");
  c10::cuda::CUDAGuard guard(img.device());
  Tensor out = at::empty_like(img);
  Tensor tmp;
  if (op == 2) tmp = at::empty({4, img.size(0), img.size(1), 4}, img.options());
  if (op == 6) tmp = at::empty({2, img.size(0), img.size(1), 4}, img.options());
  std::vector<float> p(params.begin(), params.end());
  const void* aux_ptr = nullptr;
  if (aux.has_value()) {
    TORCH_CHECK(aux->is_cuda() && aux->is_contiguous(), "image_filter: aux must be a contiguous device tensor");
    aux_ptr = aux->data_ptr();
  }
  check_rc(mdb_image_filter((int)op, img.data_ptr<float>(), out.data_ptr<float>(), tmp.defined() ? tmp.data_ptr<float>() : nullptr,
                            (int)img.size(0), (int)img.size(1), p.data(), (int)p.size(), aux_ptr, cur_stream()),
           "image_filter");
  return out;
}
Tensor upsample2x_nhwc(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "upsample2x_nhwc");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({x.size(0), x.size(1) * 2, x.size(2) * 2, x.size(3)}, x.options());
  check_rc(mdb_upsample2x(x.data_ptr(), y.data_ptr(), (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)x.size(3),
                          cur_stream()),
           "upsample2x");
  return y;
}
Tensor avgpool2x_nhwc(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 4 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "avgpool2x_nhwc");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty({x.size(0), x.size(1) / 2, x.size(2) / 2, x.size(3)}, x.options());
  check_rc(mdb_avgpool2x(x.data_ptr(), y.data_ptr(), (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)x.size(3),
                         cur_stream()),
           "avgpool2x");
  return y;
}

// ------------------------------------------------------------------------------------------
// attention
// ------------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale,
                                         const optional<Tensor>& kv_len, bool need_lse,
                                         const optional<Tensor>& out_opt, std::vector<int64_t> route_a,
                                         std::vector<int64_t> route_b, std::vector<int64_t> route_cfg) {
  // q: [B, Sq, H, Dh], k/v: [B, Skv, H, Dh] (any strides with contiguous Dh)
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && k.dim() == 4 && v.dim() == 4, "attention: [B,S,H,Dh] tensors");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "attention: bf16");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1, "attention: head dim must be contiguous");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), Sq = q.size(1), H = q.size(2), Dh = q.size(3), Skv = k.size(1);
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && k.size(2) == H && v.size(2) == H && k.size(3) == Dh &&
                  v.size(3) == Dh && v.size(1) == Skv,
              "attention: shape mismatch");
  const bool routed = !route_a.empty();
  Tensor o = (out_opt.has_value() && out_opt->defined()) ? *out_opt
             : routed ? at::empty({0}, q.options()) : at::empty({B, Sq, H, Dh}, q.options());
  TORCH_CHECK(routed || (o.dim() == 4 && o.stride(3) == 1 && o.size(1) == Sq && o.size(2) == H), "attention: bad out");
  Tensor lse;
  if (need_lse) lse = at::empty({B, H, Sq}, q.options().dtype(at::kFloat));
  MdbAttnArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr();
  a.lse = need_lse ? lse.data_ptr<float>() : nullptr;
  if (kv_len.has_value() && kv_len->defined()) {
    TORCH_CHECK(kv_len->scalar_type() == at::kInt && kv_len->numel() == B && kv_len->is_cuda(), "attention: kv_len");
    a.kv_len = kv_len->data_ptr<int>();
  }
  a.B = (int)B; a.H = (int)H; a.Sq = (int)Sq; a.Skv = (int)Skv; a.Dh = (int)Dh;
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i); a.v_strides[i] = v.stride(i);
    a.o_strides[i] = routed ? 0 : o.stride(i);
  }
  if (routed) {
    // route_cfg = {rows_a, split, rows_b, o_stride_batch, o_stride_seq, o_stride_head}
    TORCH_CHECK(route_a.size() <= 8 && route_cfg.size() == 6 && (route_b.empty() || route_b.size() == route_a.size()),
                "attention: route arguments");
    for (size_t i = 0; i < route_a.size(); ++i) {
      a.o_route_a[i] = reinterpret_cast<void*>(route_a[i]);
      a.o_route_b[i] = route_b.empty() ? nullptr : reinterpret_cast<void*>(route_b[i]);
    }
    a.route_rows_a = (int)route_cfg[0];
    a.route_split = (int)route_cfg[1];
    a.route_rows_b = (int)route_cfg[2];
    a.o_strides[0] = route_cfg[3]; a.o_strides[1] = route_cfg[4]; a.o_strides[2] = route_cfg[5];
  }
  a.scale = static_cast<float>(scale);
  a.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  a.status = status_ptr(q);
  check_rc(mdb_attention_fwd(&a, cur_stream()), "attention_fwd");
  return {o, need_lse ? lse : Tensor()};
}

std::tuple<Tensor, Tensor, Tensor> attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                                 const Tensor& lse, const Tensor& dout, double scale,
                                                 const optional<Tensor>& kv_len, std::vector<Tensor> outs) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 4 && q.scalar_type() == at::kBFloat16, "attention_bwd: [B,S,H,Dh] bf16");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && o.stride(3) == 1 && dout.stride(3) == 1,
              "attention_bwd: head dim must be contiguous");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t B = q.size(0), Sq = q.size(1), H = q.size(2), Dh = q.size(3), Skv = k.size(1);
  TORCH_CHECK(lse.scalar_type() == at::kFloat && lse.is_contiguous() && lse.numel() == B * H * Sq, "attention_bwd: lse");
  for (const Tensor* t : {&k, &v, &o, &dout})
    TORCH_CHECK(t->is_cuda() && t->device() == q.device() && t->dim() == 4 && t->scalar_type() == at::kBFloat16,
                "attention_bwd: k, v, o and dout must be [B,S,H,Dh] bf16 on q's device");
  TORCH_CHECK(lse.is_cuda() && lse.device() == q.device(), "attention_bwd: lse must be on q's device");
  TORCH_CHECK(k.size(0) == B && v.size(0) == B && k.size(2) == H && v.size(2) == H && k.size(3) == Dh && v.size(3) == Dh &&
                  v.size(1) == Skv, "attention_bwd: k / v shapes must be [B,Skv,H,Dh]");
  TORCH_CHECK(o.sizes() == q.sizes() && dout.sizes() == q.sizes(), "attention_bwd: o and dout must have q's shape");
  TORCH_CHECK(Dh == 64 || Dh == 128, "attention_bwd: head dim 64 or 128");
  if (kv_len.has_value() && kv_len->defined())
    TORCH_CHECK(kv_len->is_cuda() && kv_len->scalar_type() == at::kInt && kv_len->is_contiguous() && kv_len->numel() == B,
                "attention_bwd: kv_len must be [B] int32 on the device");
  // outs: empty, or {dq, dk, dv} views to write into (e.g. the three column ranges of one packed gradient buffer)
  TORCH_CHECK(outs.empty() || outs.size() == 3, "attention_bwd: outs must be {dq, dk, dv}");
  Tensor dq = outs.empty() ? at::empty({B, Sq, H, Dh}, q.options()) : outs[0];
  Tensor dk = outs.empty() ? at::empty({B, Skv, H, Dh}, q.options()) : outs[1];
  Tensor dv = outs.empty() ? at::empty({B, Skv, H, Dh}, q.options()) : outs[2];
  if (!outs.empty()) {
    TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes() && dq.stride(3) == 1 &&
                    dk.stride(3) == 1 && dv.stride(3) == 1 && dq.scalar_type() == at::kBFloat16 &&
                    dk.scalar_type() == at::kBFloat16 && dv.scalar_type() == at::kBFloat16,
                "attention_bwd: outs must match q / k / v with a contiguous head dim");
  }
  Tensor delta = at::empty({B, H, Sq}, lse.options());
  MdbAttnBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr(); a.dout = dout.data_ptr();
  a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr();
  a.lse = lse.data_ptr<float>();
  a.delta = delta.data_ptr<float>();
  if (kv_len.has_value() && kv_len->defined()) a.kv_len = kv_len->data_ptr<int>();
  a.B = (int)B; a.H = (int)H; a.Sq = (int)Sq; a.Skv = (int)Skv; a.Dh = (int)Dh;
  for (int i = 0; i < 3; ++i) {
    a.q_strides[i] = q.stride(i); a.k_strides[i] = k.stride(i); a.v_strides[i] = v.stride(i);
    a.o_strides[i] = o.stride(i); a.do_strides[i] = dout.stride(i);
    a.dq_strides[i] = dq.stride(i); a.dk_strides[i] = dk.stride(i); a.dv_strides[i] = dv.stride(i);
  }
  a.scale = static_cast<float>(scale);
  a.status = status_ptr(q);
  g_launches.fetch_add(2, std::memory_order_relaxed);
  check_rc(mdb_attention_bwd(&a, cur_stream()), "attention_bwd");
  return {dq, dk, dv};
}

// ------------------------------------------------------------------------------------------
// norm / rope
// ------------------------------------------------------------------------------------------
Tensor norm_modulate_fwd(const Tensor& x, const optional<Tensor>& weight, const optional<Tensor>& bias,
                         const optional<Tensor>& scale, const optional<Tensor>& shift, int64_t rows_per_group,
                         double eps, bool rms) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1, "norm: x [rows,D] bf16");
  for (const optional<Tensor>* t : {&weight, &bias, &scale, &shift})
    TORCH_CHECK(!(t->has_value() && (*t)->defined()) || (*t)->scalar_type() == at::kBFloat16, "norm: weight / bias / scale / shift must be bf16");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor out = at::empty({x.size(0), x.size(1)}, x.options());
  int mod_stride = 0;
  if (scale.has_value() && scale->defined()) {
    TORCH_CHECK(scale->dim() == 2 && scale->stride(1) == 1 && scale->size(1) == x.size(1), "norm: scale [groups,D]");
    mod_stride = (int)scale->stride(0);
    if (shift.has_value() && shift->defined())
      TORCH_CHECK(shift->stride(0) == scale->stride(0) && shift->stride(1) == 1, "norm: shift stride must match scale");
  } else if (shift.has_value() && shift->defined()) {
    mod_stride = (int)shift->stride(0);
  }
  check_rc(mdb_norm_modulate_fwd(x.data_ptr(), out.data_ptr(), opt_ptr(weight), opt_ptr(bias), opt_ptr(scale),
                                 opt_ptr(shift), nullptr, (int)x.size(0), (int)x.size(1), (int)x.stride(0),
                                 (int)out.stride(0), mod_stride, (int)rows_per_group, (float)eps, rms ? 1 : 0,
                                 cur_stream()),
           "norm_modulate_fwd");
  return out;
}

Tensor norm_modulate_bwd(const Tensor& x, const Tensor& dy, const optional<Tensor>& weight,
                         const optional<Tensor>& scale, int64_t rows_per_group, double eps, bool rms) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && dy.dim() == 2 && x.stride(1) == 1 && dy.stride(1) == 1, "norm bwd: 2-D");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty({x.size(0), x.size(1)}, x.options());
  const int mod_stride = (scale.has_value() && scale->defined()) ? (int)scale->stride(0) : 0;
  check_rc(mdb_norm_modulate_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), opt_ptr(weight), opt_ptr(scale),
                                 (int)x.size(0), (int)x.size(1), (int)x.stride(0), (int)dy.stride(0), (int)dx.stride(0),
                                 mod_stride, (int)rows_per_group, (float)eps, rms ? 1 : 0, cur_stream()),
           "norm_modulate_bwd");
  return dx;
}

// buf: [B, S, W] bf16 view (W contiguous), updated in place. q at column q_off, k at k_off, each H*Dh wide.
// Token t of the view sits at sequence position t + pos_offset of the cos/sin tables.
void qk_norm_rope(Tensor buf, const optional<Tensor>& wq, const optional<Tensor>& wk, const optional<Tensor>& cosv,
                  const optional<Tensor>& sinv, int64_t H, int64_t Dh, int64_t q_off, int64_t k_off, double eps,
                  bool interleaved, bool inverse, bool do_norm, int64_t rope_start, int64_t pos_offset) {
  TORCH_CHECK(buf.is_cuda() && buf.scalar_type() == at::kBFloat16 && buf.dim() == 3 && buf.stride(2) == 1, "qk_norm_rope: buf [B,S,W]");
  const int64_t tokens_per_batch = buf.size(1);
  c10::cuda::CUDAGuard guard(buf.device());
  if (cosv.has_value() && cosv->defined())
    TORCH_CHECK(cosv->scalar_type() == at::kFloat && cosv->is_contiguous() && cosv->size(-1) == Dh / 2,
                "qk_norm_rope: cos table [positions, Dh/2] fp32");
  if (cosv.has_value() && cosv->defined())
    TORCH_CHECK(cosv->numel() >= (tokens_per_batch + pos_offset) * (Dh / 2), "qk_norm_rope: table too short");
  check_rc(mdb_qk_norm_rope(buf.data_ptr(), opt_ptr(wq), opt_ptr(wk), (const float*)opt_ptr(cosv),
                            (const float*)opt_ptr(sinv), buf.size(0) * buf.size(1), (int)tokens_per_batch, (int)H,
                            (int)Dh, (int)buf.stride(1), (int)q_off, (int)k_off, (float)eps, interleaved, inverse,
                            do_norm, (int)rope_start, buf.stride(0), (int)pos_offset, cur_stream()),
           "qk_norm_rope");
}

void qk_norm_rope_bwd(Tensor dbuf, const Tensor& xbuf, const optional<Tensor>& wq, const optional<Tensor>& wk,
                      const optional<Tensor>& cosv, const optional<Tensor>& sinv, int64_t H, int64_t Dh, int64_t q_off,
                      int64_t k_off, double eps, bool interleaved, bool do_norm, int64_t rope_start,
                      int64_t pos_offset) {
  TORCH_CHECK(dbuf.is_cuda() && dbuf.dim() == 3 && xbuf.dim() == 3 && (dbuf.size(0) == 1 || dbuf.stride(0) == xbuf.stride(0)) &&
                  dbuf.stride(1) == xbuf.stride(1) && dbuf.stride(2) == 1 && xbuf.stride(2) == 1,
              "qk_norm_rope_bwd: [B,S,W] views with equal strides");
  const int64_t tokens_per_batch = dbuf.size(1);
  c10::cuda::CUDAGuard guard(dbuf.device());
  check_rc(mdb_qk_norm_rope_bwd(dbuf.data_ptr(), xbuf.data_ptr(), opt_ptr(wq), opt_ptr(wk), (const float*)opt_ptr(cosv),
                                (const float*)opt_ptr(sinv), dbuf.size(0) * dbuf.size(1), (int)tokens_per_batch, (int)H,
                                (int)Dh, (int)dbuf.stride(1), (int)q_off, (int)k_off, (float)eps, interleaved, do_norm,
                                (int)rope_start, dbuf.stride(0), (int)pos_offset, cur_stream()),
           "qk_norm_rope_bwd");
}

std::tuple<Tensor, Tensor> rope_table(const Tensor& pos, std::vector<int64_t> axes_dim, double theta) {
  TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == at::kFloat && pos.dim() == 2 && pos.is_contiguous(), "rope_table: pos [T, axes] fp32");
  c10::cuda::CUDAGuard guard(pos.device());
  TORCH_CHECK((int64_t)axes_dim.size() == pos.size(1), "rope_table: axes");
  int ad[4] = {0, 0, 0, 0};
  int64_t half = 0;
  for (size_t i = 0; i < axes_dim.size(); ++i) {
    ad[i] = (int)axes_dim[i];
    half += axes_dim[i] / 2;
  }
  Tensor c = at::empty({pos.size(0), half}, pos.options());
  Tensor s = at::empty({pos.size(0), half}, pos.options());
  check_rc(mdb_rope_table(pos.data_ptr<float>(), c.data_ptr<float>(), s.data_ptr<float>(), (int)pos.size(0),
                          (int)axes_dim.size(), ad, (float)theta, cur_stream()),
           "rope_table");
  return {c, s};
}

// ------------------------------------------------------------------------------------------
// pointwise
// ------------------------------------------------------------------------------------------
Tensor act_fwd(const Tensor& x, const optional<Tensor>& bias, int64_t act) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous(), "act_fwd: contiguous bf16");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor y = at::empty_like(x);
  check_rc(mdb_act_fwd(x.data_ptr(), y.data_ptr(), opt_ptr(bias), x.numel(), (int)x.size(-1), (int)act, cur_stream()), "act_fwd");
  return y;
}
Tensor act_bwd(const Tensor& x, const Tensor& dy, const optional<Tensor>& bias, int64_t act) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && dy.is_contiguous() && x.scalar_type() == at::kBFloat16, "act_bwd");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty_like(x);
  check_rc(mdb_act_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), opt_ptr(bias), x.numel(), (int)x.size(-1), (int)act,
                       cur_stream()),
           "act_bwd");
  return dx;
}
Tensor glu_fwd(const Tensor& x, int64_t act, bool second) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16, "glu_fwd");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t F = x.size(1) / 2;
  Tensor y = at::empty({x.size(0), F}, x.options());
  check_rc(mdb_glu_fwd(x.data_ptr(), y.data_ptr(), x.size(0), (int)F, (int)x.stride(0), (int)y.stride(0), (int)act, second,
                       cur_stream()),
           "glu_fwd");
  return y;
}
Tensor glu_bwd(const Tensor& x, const Tensor& dy, int64_t act, bool second) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && dy.dim() == 2 && x.stride(1) == 1 && dy.stride(1) == 1, "glu_bwd");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor dx = at::empty({x.size(0), x.size(1)}, x.options());
  check_rc(mdb_glu_bwd(x.data_ptr(), dy.data_ptr(), dx.data_ptr(), x.size(0), (int)(x.size(1) / 2), (int)x.stride(0),
                       (int)dy.stride(0), (int)dx.stride(0), (int)act, second, cur_stream()),
           "glu_bwd");
  return dx;
}
Tensor gate_residual(const Tensor& x, const Tensor& y, const optional<Tensor>& gate, int64_t rows_per_group,
                     bool tanh_gate) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && y.is_contiguous() && x.scalar_type() == at::kBFloat16, "gate_residual");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t D = x.size(-1);
  Tensor out = at::empty_like(x);
  int gs = 0;
  if (gate.has_value() && gate->defined()) {
    TORCH_CHECK(gate->dim() == 2 && gate->stride(1) == 1 && gate->size(1) == D, "gate_residual: gate [groups,D]");
    gs = (int)gate->stride(0);
  }
  check_rc(mdb_gate_residual(x.data_ptr(), y.data_ptr(), opt_ptr(gate), out.data_ptr(), x.numel() / D, (int)D, gs,
                             (int)rows_per_group, tanh_gate, cur_stream()),
           "gate_residual");
  return out;
}
// out[rows, cols] = act(x) (dy absent) or dy * act'(x), on row-strided 2-D views; act 0 without dy is a strided copy
void act_strided(const Tensor& x, const optional<Tensor>& dy, Tensor out, int64_t act) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 &&
                  x.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 && x.sizes() == out.sizes() &&
                  out.device() == x.device(),
              "act_strided: bf16 [rows, cols] views with a contiguous last dimension");
  const bool has_dy = dy.has_value() && dy->defined();
  if (has_dy)
    TORCH_CHECK(dy->dim() == 2 && dy->stride(1) == 1 && dy->sizes() == x.sizes() && dy->scalar_type() == at::kBFloat16 &&
                    dy->device() == x.device(),
                "act_strided: dy must match x");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(mdb_act_strided(x.data_ptr(), x.stride(0), has_dy ? dy->data_ptr() : nullptr, has_dy ? dy->stride(0) : 0,
                           out.data_ptr(), out.stride(0), x.size(0), (int)x.size(1), (int)act, cur_stream()),
           "act_strided");
}
// gated linear unit on row-strided views: out[rows, F] = glu(x[rows, 2F]) (dy absent) or out[rows, 2F] = its gradient
void glu_strided(const Tensor& x, const optional<Tensor>& dy, Tensor out, int64_t act, bool second) {
  const bool has_dy = dy.has_value() && dy->defined();
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && out.dim() == 2 && x.stride(1) == 1 && out.stride(1) == 1 &&
                  x.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 && x.size(1) % 16 == 0 &&
                  out.size(0) == x.size(0) && out.size(1) == (has_dy ? x.size(1) : x.size(1) / 2) &&
                  out.device() == x.device(),
              "glu_strided: bf16 [rows, 2F] input view, [rows, F] (forward) or [rows, 2F] (gradient) output view");
  const int64_t F = x.size(1) / 2;
  if (has_dy)
    TORCH_CHECK(dy->dim() == 2 && dy->stride(1) == 1 && dy->size(0) == x.size(0) && dy->size(1) == F &&
                    dy->scalar_type() == at::kBFloat16 && dy->device() == x.device(),
                "glu_strided: dy [rows, F]");
  TORCH_CHECK(reinterpret_cast<uintptr_t>(x.data_ptr()) % 16 == 0 && reinterpret_cast<uintptr_t>(out.data_ptr()) % 16 == 0,
              "glu_strided: 16-byte aligned views");
  if (has_dy) TORCH_CHECK(reinterpret_cast<uintptr_t>(dy->data_ptr()) % 16 == 0, "glu_strided: 16-byte aligned dy");
  c10::cuda::CUDAGuard guard(x.device());
  if (has_dy)
    check_rc(mdb_glu_bwd(x.data_ptr(), dy->data_ptr(), out.data_ptr(), x.size(0), (int)F, (int)x.stride(0),
                         (int)dy->stride(0), (int)out.stride(0), (int)act, second, cur_stream()),
             "glu_strided (gradient)");
  else
    check_rc(mdb_glu_fwd(x.data_ptr(), out.data_ptr(), x.size(0), (int)F, (int)x.stride(0), (int)out.stride(0), (int)act,
                         second, cur_stream()),
             "glu_strided");
}
// dy = gate[group] * dout: the gradient of the gated branch of gate_residual
Tensor gate_mul(const Tensor& y, const Tensor& gate, int64_t rows_per_group, bool tanh_gate) {
  TORCH_CHECK(y.is_cuda() && y.is_contiguous() && y.scalar_type() == at::kBFloat16, "gate_mul: contiguous bf16");
  c10::cuda::CUDAGuard guard(y.device());
  const int64_t D = y.size(-1);
  TORCH_CHECK(gate.dim() == 2 && gate.stride(1) == 1 && gate.size(1) == D && gate.scalar_type() == at::kBFloat16 &&
                  gate.device() == y.device(),
              "gate_mul: gate [groups, D] bf16");
  Tensor out = at::empty_like(y);
  check_rc(mdb_gate_residual(nullptr, y.data_ptr(), gate.data_ptr(), out.data_ptr(), y.numel() / D, (int)D,
                             (int)gate.stride(0), (int)rows_per_group, tanh_gate, cur_stream()),
           "gate_mul");
  return out;
}
void cfg_euler(Tensor x, const Tensor& vc, const optional<Tensor>& vu, const optional<Tensor>& x_bf16, double dt,
               double s, int64_t mode) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kFloat && x.is_contiguous() && vc.is_contiguous() &&
                  vc.scalar_type() == at::kBFloat16 && vc.numel() == x.numel(),
              "cfg_euler");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(mdb_cfg_euler(x.data_ptr<float>(), vc.data_ptr(), opt_ptr(vu),
                         x_bf16.has_value() && x_bf16->defined() ? x_bf16->data_ptr() : nullptr, x.numel(), (float)dt,
                         (float)s, (int)mode, cur_stream()),
           "cfg_euler");
}
std::tuple<Tensor, Tensor> flow_match(const Tensor& x0, const Tensor& eps, const Tensor& sigma) {
  TORCH_CHECK(x0.is_cuda() && x0.scalar_type() == at::kFloat && eps.scalar_type() == at::kFloat &&
                  sigma.scalar_type() == at::kFloat && x0.is_contiguous() && eps.is_contiguous(),
              "flow_match: fp32 contiguous");
  c10::cuda::CUDAGuard guard(x0.device());
  Tensor xt = at::empty_like(x0, x0.options().dtype(at::kBFloat16));
  Tensor tgt = at::empty_like(x0);
  check_rc(mdb_flow_match(x0.data_ptr<float>(), eps.data_ptr<float>(), sigma.data_ptr<float>(), xt.data_ptr(),
                          tgt.data_ptr<float>(), x0.numel(), x0.numel() / x0.size(0), cur_stream()),
           "flow_match");
  return {xt, tgt};
}
std::tuple<Tensor, Tensor> mse_loss(const Tensor& pred, const Tensor& target, bool need_grad, double grad_scale) {
  TORCH_CHECK(pred.is_cuda() && pred.scalar_type() == at::kBFloat16 && target.scalar_type() == at::kFloat &&
                  pred.is_contiguous() && target.is_contiguous() && pred.numel() == target.numel(),
              "mse_loss");
  c10::cuda::CUDAGuard guard(pred.device());
  Tensor sum = at::zeros({}, target.options());
  Tensor grad;
  if (need_grad) grad = at::empty_like(pred);
  const double n = (double)pred.numel();
  check_rc(mdb_mse_loss(pred.data_ptr(), target.data_ptr<float>(), need_grad ? grad.data_ptr() : nullptr,
                        sum.data_ptr<float>(), pred.numel(), (float)(2.0 / n * grad_scale), cur_stream()),
           "mse_loss");
  return {sum / n, grad};
}
Tensor randn(std::vector<int64_t> shape, int64_t seed, int64_t offset, bool bf16, const Tensor& like) {
  c10::cuda::CUDAGuard guard(like.device());
  Tensor out = at::empty(shape, like.options().dtype(bf16 ? at::kBFloat16 : at::kFloat));
  check_rc(mdb_randn(bf16 ? nullptr : out.data_ptr<float>(), bf16 ? out.data_ptr() : nullptr, out.numel(),
                     (unsigned long long)seed, (unsigned long long)offset, cur_stream()),
           "randn");
  return out;
}
std::tuple<Tensor, Tensor> fp8_quant_rows(const Tensor& x) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16, "fp8_quant_rows");
  c10::cuda::CUDAGuard guard(x.device());
  Tensor q = at::empty({x.size(0), x.size(1)}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor sc = at::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check_rc(mdb_fp8_quant_rows(x.data_ptr(), q.data_ptr(), sc.data_ptr<float>(), x.size(0), (int)x.size(1),
                              (int)x.stride(0), (int)q.stride(0), cur_stream()),
           "fp8_quant_rows");
  return {q, sc};
}
Tensor fp8_dequant(const Tensor& q, const optional<Tensor>& row_scale, double tensor_scale) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 2 && q.is_contiguous() && q.scalar_type() == at::kFloat8_e4m3fn, "fp8_dequant");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor y = at::empty({q.size(0), q.size(1)}, q.options().dtype(at::kBFloat16));
  check_rc(mdb_fp8_dequant(q.data_ptr(), (const float*)opt_ptr(row_scale), (float)tensor_scale, y.data_ptr(), q.size(0),
                           (int)q.size(1), cur_stream()),
           "fp8_dequant");
  return y;
}

// rows -> (E4M3 bytes [rows, K], scale chunks padded to ``pad_rows`` rows per tile row)
std::tuple<Tensor, Tensor> mxfp8_quant_rows(const Tensor& x, int64_t pad_rows) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1 && x.scalar_type() == at::kBFloat16 && x.size(1) % 128 == 0,
              "mxfp8_quant_rows: bf16 [rows, K] with contiguous K, K a multiple of 128");
  TORCH_CHECK(pad_rows == 128 || pad_rows == 256, "mxfp8_quant_rows: pad_rows 128 (A operand) or 256 (B operand)");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t rows = x.size(0), K = x.size(1);
  const int64_t padded = (rows + pad_rows - 1) / pad_rows * pad_rows;
  Tensor q = at::empty({rows, K}, x.options().dtype(at::kByte));
  Tensor sf = at::full({padded / 128, K / 128, 512}, 127, x.options().dtype(at::kByte));
  check_rc(mdb_mxfp8_quant_rows(x.data_ptr(), q.data_ptr(), sf.data_ptr(), rows, (int)K, x.stride(0), cur_stream()), "mxfp8_quant_rows");
  return {q, sf};
}
Tensor gemm_mxfp8(const Tensor& a_q, const Tensor& sfa, const Tensor& b_q, const Tensor& sfb, const optional<Tensor>& bias) {
  TORCH_CHECK(a_q.is_cuda() && a_q.dim() == 2 && a_q.is_contiguous() && a_q.scalar_type() == at::kByte, "gemm_mxfp8: a_q uint8 [M, K]");
  TORCH_CHECK(b_q.is_cuda() && b_q.dim() == 2 && b_q.is_contiguous() && b_q.scalar_type() == at::kByte && b_q.size(1) == a_q.size(1) &&
                  b_q.device() == a_q.device(), "gemm_mxfp8: b_q uint8 [N, K]");
  const int64_t M = a_q.size(0), N = b_q.size(0), K = a_q.size(1);
  TORCH_CHECK(K % 128 == 0 && N % 8 == 0, "gemm_mxfp8: K a multiple of 128, N a multiple of 8");
  TORCH_CHECK(sfa.is_cuda() && sfa.is_contiguous() && sfa.scalar_type() == at::kByte && sfa.numel() == (M + 127) / 128 * (K / 128) * 512,
              "gemm_mxfp8: sfa must hold ceil(M/128) x K/128 chunks of 512 bytes");
  TORCH_CHECK(sfb.is_cuda() && sfb.is_contiguous() && sfb.scalar_type() == at::kByte && sfb.numel() == (N + 255) / 256 * 2 * (K / 128) * 512,
              "gemm_mxfp8: sfb must hold 2 * ceil(N/256) x K/128 chunks of 512 bytes");
  if (bias.has_value() && bias->defined())
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kBFloat16 && bias->is_contiguous() && bias->numel() == N, "gemm_mxfp8: bias bf16 [N]");
  c10::cuda::CUDAGuard guard(a_q.device());
  Tensor out = at::empty({M, N}, a_q.options().dtype(at::kBFloat16));
  g_launches.fetch_add(1, std::memory_order_relaxed);
  check_rc(mdb_gemm_mxfp8(a_q.data_ptr(), sfa.data_ptr(), b_q.data_ptr(), sfb.data_ptr(), out.data_ptr(), opt_ptr(bias), (int)M, (int)N,
                          (int)K, (int)N, status_ptr(a_q), cur_stream()), "gemm_mxfp8");
  return out;
}
Tensor mx_dequant(const Tensor& q, const Tensor& scales, bool fp4) {
  TORCH_CHECK(q.is_cuda() && q.is_contiguous() && q.scalar_type() == at::kByte && scales.is_cuda() && scales.is_contiguous() &&
                  scales.scalar_type() == at::kByte && scales.device() == q.device(), "mx_dequant: uint8 device tensors");
  const int64_t per = fp4 ? 16 : 32, nb = scales.numel();
  TORCH_CHECK(q.numel() == nb * per, "mx_dequant: ", per, " bytes per 32-element block and one scale byte per block");
  c10::cuda::CUDAGuard guard(q.device());
  Tensor y = at::empty({nb * 32}, q.options().dtype(at::kBFloat16));
  check_rc(mdb_mx_dequant(q.data_ptr(), scales.data_ptr(), y.data_ptr(), nb, fp4 ? 1 : 0, cur_stream()), "mx_dequant");
  return y;
}
std::tuple<Tensor, Tensor> mx_quant(const Tensor& x, bool fp4) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 && x.numel() % 32 == 0,
              "mx_quant: contiguous bf16 with a multiple of 32 elements");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t nb = x.numel() / 32;
  Tensor q = at::empty({nb * (fp4 ? 16 : 32)}, x.options().dtype(at::kByte));
  Tensor sc = at::empty({nb}, x.options().dtype(at::kByte));
  check_rc(mdb_mx_quant(x.data_ptr(), q.data_ptr(), sc.data_ptr(), nb, fp4 ? 1 : 0, cur_stream()), "mx_quant");
  return {q, sc};
}

// ------------------------------------------------------------------------------------------
// optimizer (tables are int64 device tensors laid out as MdbTensorEntry / int2)
// ------------------------------------------------------------------------------------------
void adamw_multi(const Tensor& table, const Tensor& chunks, int64_t chunk_elems, bool p_bf16, bool g_bf16, bool m_bf16,
                 double lr, double beta1, double beta2, double eps, double wd, int64_t step, double grad_scale,
                 const optional<Tensor>& norm_sq, double max_norm, int64_t seed, bool stochastic) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.size(-1) == 6, "adamw: table [n,6] int64");
  TORCH_CHECK(chunks.is_cuda() && chunks.scalar_type() == at::kInt && chunks.is_contiguous() && chunks.size(-1) == 2, "adamw: chunks [c,2] int32");
  c10::cuda::CUDAGuard guard(table.device());
  check_rc(mdb_adamw_multi((const MdbTensorEntry*)table.data_ptr(), chunks.data_ptr<int>(), (int)chunks.size(0),
                           (int)chunk_elems, p_bf16, g_bf16, m_bf16, (float)lr, (float)beta1, (float)beta2, (float)eps,
                           (float)wd, (int)step, (float)grad_scale, (const float*)opt_ptr(norm_sq), (float)max_norm,
                           (unsigned int)seed, stochastic, status_ptr(table), cur_stream()),
           "adamw_multi");
}
void lion_multi(const Tensor& table, const Tensor& chunks, int64_t chunk_elems, bool p_bf16, bool g_bf16, double lr,
                double beta1, double beta2, double wd, double grad_scale) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.size(-1) == 6, "lion: table [n,6] int64");
  TORCH_CHECK(chunks.is_cuda() && chunks.scalar_type() == at::kInt && chunks.is_contiguous() && chunks.size(-1) == 2, "lion: chunks [c,2] int32");
  c10::cuda::CUDAGuard guard(table.device());
  check_rc(mdb_lion_multi((const MdbTensorEntry*)table.data_ptr(), chunks.data_ptr<int>(), (int)chunks.size(0), (int)chunk_elems,
                          p_bf16, g_bf16, (float)lr, (float)beta1, (float)beta2, (float)wd, (float)grad_scale,
                          status_ptr(table), cur_stream()),
           "lion_multi");
}
// beta1h / beta2h: the debiased betas of this step; returns the per-tensor sums of g^2 / max(v, eps^2)
Tensor stable_adamw_multi(const Tensor& table, const Tensor& chunks, int64_t chunk_elems, bool p_bf16, bool g_bf16, double lr,
                          double beta1h, double beta2h, double eps, double wd, double grad_scale) {
  TORCH_CHECK(table.is_cuda() && table.scalar_type() == at::kLong && table.is_contiguous() && table.size(-1) == 6, "stable_adamw: table [n,6] int64");
  TORCH_CHECK(chunks.is_cuda() && chunks.scalar_type() == at::kInt && chunks.is_contiguous() && chunks.size(-1) == 2, "stable_adamw: chunks [c,2] int32");
  c10::cuda::CUDAGuard guard(table.device());
  Tensor acc = at::zeros({table.size(0)}, table.options().dtype(at::kFloat));
  check_rc(mdb_stable_adamw_multi((const MdbTensorEntry*)table.data_ptr(), chunks.data_ptr<int>(), (int)chunks.size(0),
                                  (int)chunk_elems, p_bf16, g_bf16, (float)lr, (float)beta1h, (float)beta2h, (float)eps,
                                  (float)wd, (float)grad_scale, acc.data_ptr<float>(), status_ptr(table), cur_stream()),
           "stable_adamw_multi");
  return acc;
}
Tensor sumsq_multi(const Tensor& table, const Tensor& chunks, int64_t chunk_elems, bool g_bf16) {
  c10::cuda::CUDAGuard guard(table.device());
  Tensor out = at::zeros({}, table.options().dtype(at::kFloat));
  check_rc(mdb_sumsq_multi((const MdbTensorEntry*)table.data_ptr(), chunks.data_ptr<int>(), (int)chunks.size(0),
                           (int)chunk_elems, g_bf16, out.data_ptr<float>(), cur_stream()),
           "sumsq_multi");
  return out;
}
void ema_multi(const Tensor& table, const Tensor& chunks, int64_t chunk_elems, bool p_bf16, double decay) {
  c10::cuda::CUDAGuard guard(table.device());
  check_rc(mdb_ema_multi((const MdbTensorEntry*)table.data_ptr(), chunks.data_ptr<int>(), (int)chunks.size(0),
                         (int)chunk_elems, p_bf16, (float)decay, cur_stream()),
           "ema_multi");
}

void adamw8bit(Tensor p, const Tensor& g, Tensor qm, Tensor qv, Tensor am, Tensor av, const Tensor& code_s,
               const Tensor& code_u, double lr, double b1, double b2, double eps, double wd, int64_t step, double grad_scale) {
  c10::cuda::CUDAGuard guard(p.device());
  const int64_t n = p.numel();
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && g.numel() == n, "adamw8bit: contiguous p / g of one size");
  TORCH_CHECK(qm.scalar_type() == at::kByte && qv.scalar_type() == at::kByte && qm.numel() == n && qv.numel() == n, "adamw8bit: codes");
  TORCH_CHECK(am.scalar_type() == at::kFloat && av.scalar_type() == at::kFloat && am.numel() == (n + 255) / 256 && av.numel() == am.numel(),
              "adamw8bit: one fp32 maximum per 256 elements");
  TORCH_CHECK(code_s.scalar_type() == at::kFloat && code_s.numel() == 256 && code_u.scalar_type() == at::kFloat && code_u.numel() == 256,
              "adamw8bit: 256-entry code books");
  const bool pb = p.scalar_type() == at::kBFloat16, gb = g.scalar_type() == at::kBFloat16;
  TORCH_CHECK((pb || p.scalar_type() == at::kFloat) && (gb || g.scalar_type() == at::kFloat), "adamw8bit: bf16 or fp32");
  check_rc(mdb_adamw8bit(p.data_ptr(), g.data_ptr(), qm.data_ptr(), qv.data_ptr(), am.data_ptr<float>(), av.data_ptr<float>(),
                         code_s.data_ptr<float>(), code_u.data_ptr<float>(), n, pb, gb, (float)lr, (float)b1, (float)b2,
                         (float)eps, (float)wd, (int)step, (float)grad_scale, cur_stream()),
           "adamw8bit");
}

// ------------------------------------------------------------------------------------------
// peer-memory communication (addresses come from symmetric-memory handles: one entry per rank)
// ------------------------------------------------------------------------------------------
MdbPeerTable peer_table(const std::vector<int64_t>& ptrs) {
  TORCH_CHECK(!ptrs.empty() && ptrs.size() <= MDB_MAX_RANKS, "peer table: 1..8 ranks");
  MdbPeerTable t;
  memset(&t, 0, sizeof(t));
  for (size_t i = 0; i < ptrs.size(); ++i) t.p[i] = reinterpret_cast<void*>(ptrs[i]);
  return t;
}
void flag_signal(std::vector<int64_t> flag_ptrs, int64_t slot, int64_t rank, int64_t value, const Tensor& like,
                 const optional<Tensor>& counters) {
  c10::cuda::CUDAGuard guard(like.device());
  MdbPeerTable f = peer_table(flag_ptrs);
  int* c = counters.has_value() && counters->defined() ? counters->data_ptr<int>() : nullptr;
  check_rc(mdb_flag_signal(&f, (int)slot, (int)rank, (int)flag_ptrs.size(), (int)value, c, cur_stream()), "flag_signal");
}
void flag_wait(const Tensor& my_flags, int64_t slot, int64_t world, int64_t value, const optional<Tensor>& counters) {
  c10::cuda::CUDAGuard guard(my_flags.device());
  int* c = counters.has_value() && counters->defined() ? counters->data_ptr<int>() : nullptr;
  check_rc(mdb_flag_wait(my_flags.data_ptr<int>(), (int)slot, (int)world, (int)value, c, status_ptr(my_flags),
                         cur_stream()),
           "flag_wait");
}
void flag_barrier(std::vector<int64_t> flag_ptrs, const Tensor& my_flags, int64_t slot, int64_t rank, int64_t value,
                  const optional<Tensor>& counters) {
  c10::cuda::CUDAGuard guard(my_flags.device());
  MdbPeerTable f = peer_table(flag_ptrs);
  int* c = counters.has_value() && counters->defined() ? counters->data_ptr<int>() : nullptr;
  check_rc(mdb_flag_barrier(&f, my_flags.data_ptr<int>(), (int)slot, (int)rank, (int)flag_ptrs.size(), (int)value, c,
                            status_ptr(my_flags), cur_stream()),
           "flag_barrier");
}
Tensor rs_finalize(std::vector<int64_t> flag_ptrs, const Tensor& my_flags, int64_t slot, int64_t epoch, int64_t rank,
                   const Tensor& stage, const optional<Tensor>& bias, const optional<Tensor>& residual,
                   const optional<Tensor>& gate, int64_t rows_per_group, const optional<Tensor>& accum) {
  TORCH_CHECK(stage.is_cuda() && stage.dim() == 3 && stage.is_contiguous() && stage.scalar_type() == at::kBFloat16,
              "rs_finalize: stage must be bf16 [world, rows, D]");
  TORCH_CHECK((int64_t)flag_ptrs.size() == stage.size(0), "rs_finalize: one staging slot per rank");
  c10::cuda::CUDAGuard guard(stage.device());
  MdbPeerTable f = peer_table(flag_ptrs);
  Tensor out;
  float* acc_ptr = nullptr;
  if (accum.has_value() && accum->defined()) {
    TORCH_CHECK(accum->scalar_type() == at::kFloat && accum->is_contiguous() && accum->numel() == stage.size(1) * stage.size(2),
                "rs_finalize: accum must be fp32 [rows, D]");
    acc_ptr = accum->data_ptr<float>();
    out = *accum;
  } else {
    out = at::empty({stage.size(1), stage.size(2)}, stage.options());
  }
  int64_t gate_stride = 0;
  if (gate.has_value()) {
    TORCH_CHECK(gate->dim() == 2 && gate->stride(1) == 1 && gate->size(1) == stage.size(2), "rs_finalize: gate [groups, D]");
    gate_stride = gate->stride(0);
  }
  if (residual.has_value()) TORCH_CHECK(residual->is_contiguous() && residual->numel() == stage.size(1) * stage.size(2), "rs_finalize: residual");
  check_rc(mdb_rs_finalize(&f, my_flags.data_ptr<int>(), (int)slot, (int)epoch, (int)rank, (int)stage.size(0), stage.data_ptr(),
                           stage.size(1), (int)stage.size(2), opt_ptr(bias), opt_ptr(residual), opt_ptr(gate),
                           (int)rows_per_group, gate_stride, acc_ptr ? nullptr : out.data_ptr(), acc_ptr, status_ptr(stage),
                           cur_stream()),
           "rs_finalize");
  return out;
}
void rs_adamw(std::vector<int64_t> flag_ptrs, const Tensor& my_flags, int64_t slot, int64_t epoch, int64_t rank, const Tensor& stage,
              Tensor master, Tensor m, Tensor v, Tensor shadow, double lr, double beta1, double beta2, double eps, double wd, int64_t step,
              double grad_scale) {
  TORCH_CHECK(stage.is_cuda() && stage.dim() == 3 && stage.is_contiguous() && stage.scalar_type() == at::kBFloat16, "rs_adamw: stage bf16 [world, rows, D]");
  TORCH_CHECK((int64_t)flag_ptrs.size() == stage.size(0), "rs_adamw: one staging slot per rank");
  const int64_t n = stage.size(1) * stage.size(2);
  for (const Tensor* t : {&master, &m, &v})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n && t->device() == stage.device(),
                "rs_adamw: master / m / v must be fp32 [rows, D] on the stage's device");
  TORCH_CHECK(shadow.scalar_type() == at::kBFloat16 && shadow.is_contiguous() && shadow.numel() == n && shadow.device() == stage.device(),
              "rs_adamw: shadow must be bf16 [rows, D]");
  c10::cuda::CUDAGuard guard(stage.device());
  MdbPeerTable f = peer_table(flag_ptrs);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  check_rc(mdb_rs_adamw(&f, my_flags.data_ptr<int>(), (int)slot, (int)epoch, (int)rank, (int)stage.size(0), stage.data_ptr(), n,
                        master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(), shadow.data_ptr(), (float)lr, (float)beta1,
                        (float)beta2, (float)eps, (float)wd, (int)step, (float)grad_scale, status_ptr(stage), cur_stream()),
           "rs_adamw");
}
void peer_gather(std::vector<int64_t> src_ptrs, Tensor dst, int64_t chunk_bytes, int64_t rank, bool copy_local) {
  c10::cuda::CUDAGuard guard(dst.device());
  MdbPeerTable s = peer_table(src_ptrs);
  TORCH_CHECK(dst.is_contiguous() && dst.numel() * dst.element_size() >= chunk_bytes * (int64_t)src_ptrs.size(), "peer_gather: dst too small");
  check_rc(mdb_peer_gather(&s, dst.data_ptr(), chunk_bytes, (int)rank, (int)src_ptrs.size(), copy_local, cur_stream()),
           "peer_gather");
}
void dp_reduce_shard(std::vector<int64_t> grad_ptrs, int64_t grads_mc, const Tensor& my_flags, int64_t ready_slot,
                     int64_t epoch, int64_t lo, int64_t hi, Tensor red, Tensor sumsq) {
  c10::cuda::CUDAGuard guard(red.device());
  MdbPeerTable g = peer_table(grad_ptrs);
  TORCH_CHECK(red.scalar_type() == at::kFloat && red.numel() >= hi - lo && sumsq.scalar_type() == at::kFloat, "dp_reduce_shard");
  check_rc(mdb_dp_reduce_shard(&g, reinterpret_cast<const void*>(grads_mc), my_flags.data_ptr<int>(), (int)ready_slot,
                               (int)epoch, (int)grad_ptrs.size(), lo, hi, red.data_ptr<float>(), sumsq.data_ptr<float>(),
                               status_ptr(red), cur_stream()),
           "dp_reduce_shard");
}
void publish_scalar(std::vector<int64_t> scalar_ptrs, std::vector<int64_t> flag_ptrs, const Tensor& value, int64_t slot,
                    int64_t rank, int64_t epoch) {
  c10::cuda::CUDAGuard guard(value.device());
  MdbPeerTable sc = peer_table(scalar_ptrs), f = peer_table(flag_ptrs);
  check_rc(mdb_publish_scalar(&sc, &f, value.data_ptr<float>(), (int)slot, (int)rank, (int)flag_ptrs.size(), (int)epoch,
                              status_ptr(value), cur_stream()),
           "publish_scalar");
}
void dp_adamw_shard(std::vector<int64_t> param_ptrs, int64_t params_mc, std::vector<int64_t> flag_ptrs,
                    const Tensor& my_flags, const Tensor& my_scalars, int64_t norm_slot, int64_t done_slot, int64_t epoch,
                    int64_t rank, int64_t lo, int64_t hi, const Tensor& red, Tensor m, Tensor v, double lr, double beta1,
                    double beta2, double eps, double wd, int64_t step, double grad_scale, double max_norm, Tensor norm_out,
                    Tensor done_counter) {
  c10::cuda::CUDAGuard guard(red.device());
  MdbPeerTable p = peer_table(param_ptrs), f = peer_table(flag_ptrs);
  check_rc(mdb_dp_adamw_shard(&p, reinterpret_cast<void*>(params_mc), &f, my_flags.data_ptr<int>(),
                              my_scalars.data_ptr<float>(), (int)norm_slot, (int)done_slot, (int)epoch, (int)rank,
                              (int)param_ptrs.size(), lo, hi, red.data_ptr<float>(), m.data_ptr<float>(),
                              v.data_ptr<float>(), (float)lr, (float)beta1, (float)beta2, (float)eps, (float)wd, (int)step,
                              (float)grad_scale, (float)max_norm, norm_out.data_ptr<float>(), done_counter.data_ptr<int>(),
                              status_ptr(red), cur_stream()),
           "dp_adamw_shard");
}

// ------------------------------------------------------------------------------------------
// status
// ------------------------------------------------------------------------------------------
std::vector<int64_t> read_status(const Tensor& like, bool reset) {
  int* p = status_ptr(like);
  int h[4];
  C10_CUDA_CHECK(cudaMemcpy(h, p, sizeof(h), cudaMemcpyDeviceToHost));
  if (reset && h[0] != 0) C10_CUDA_CHECK(cudaMemset(p, 0, sizeof(h)));
  return {h[0], h[1], h[2], h[3]};
}

void attention_set_trace(const optional<Tensor>& trace) {
  if (trace.has_value() && trace->defined()) {
    TORCH_CHECK(trace->is_cuda() && trace->scalar_type() == at::kLong && trace->is_contiguous() && trace->numel() % 4 == 0, "attention_set_trace: int64 [4, len]");
    mdb_attention_set_trace(reinterpret_cast<long long*>(trace->data_ptr()), (int)(trace->numel() / 4));
  } else {
    mdb_attention_set_trace(nullptr, 0);
  }
}

// limit of every bounded device-side wait on the current device, in nanoseconds (default 1e9)
void set_wait_limit_ns(int64_t ns) {
  TORCH_CHECK(ns > 0, "set_wait_limit_ns: positive nanoseconds");
  const unsigned long long v = static_cast<unsigned long long>(ns);
  const int rc = mdb_set_wait_limit_gemm(v) | mdb_set_wait_limit_attn_fwd(v) | mdb_set_wait_limit_attn_bwd(v) |
                 mdb_set_wait_limit_comm(v) | mdb_set_wait_limit_mxfp8(v);
  TORCH_CHECK(rc == 0, "set_wait_limit_ns failed: ", rc);
}

// number of kernel launches issued through this library since load
int64_t launch_count() { return g_launches.load(); }
int64_t gemm_pair_capacity() { return mdb_gemm_pair_capacity(at::cuda::getCurrentDeviceProperties()->multiProcessorCount); }

}  // namespace

TORCH_LIBRARY(mdb200, m) {
  m.def("launch_count", &launch_count);
  m.def("gemm_pair_capacity", &gemm_pair_capacity);
  m.def("gemm", &gemm);
  m.def("conv2d_nhwc", &conv2d_nhwc);
  m.def("group_norm_nhwc", &group_norm_nhwc);
  m.def("group_norm_nhwc_bwd", &group_norm_nhwc_bwd);
  m.def("image_filter", &image_filter);
  m.def("upsample2x_nhwc", &upsample2x_nhwc);
  m.def("avgpool2x_nhwc", &avgpool2x_nhwc);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
  m.def("norm_modulate_fwd", &norm_modulate_fwd);
  m.def("norm_modulate_bwd", &norm_modulate_bwd);
  m.def("qk_norm_rope", &qk_norm_rope);
  m.def("qk_norm_rope_bwd", &qk_norm_rope_bwd);
  m.def("rope_table", &rope_table);
  m.def("act_fwd", &act_fwd);
  m.def("act_bwd", &act_bwd);
  m.def("glu_fwd", &glu_fwd);
  m.def("glu_bwd", &glu_bwd);
  m.def("gate_residual", &gate_residual);
  m.def("gate_mul", &gate_mul);
  m.def("act_strided", &act_strided);
  m.def("glu_strided", &glu_strided);
  m.def("cfg_euler", &cfg_euler);
  m.def("flow_match", &flow_match);
  m.def("mse_loss", &mse_loss);
  m.def("randn", &randn);
  m.def("fp8_quant_rows", &fp8_quant_rows);
  m.def("fp8_dequant", &fp8_dequant);
  m.def("mx_dequant", &mx_dequant);
  m.def("mxfp8_quant_rows", &mxfp8_quant_rows);
  m.def("gemm_mxfp8", &gemm_mxfp8);
  m.def("mx_quant", &mx_quant);
  m.def("adamw_multi", &adamw_multi);
  m.def("lion_multi", &lion_multi);
  m.def("stable_adamw_multi", &stable_adamw_multi);
  m.def("sumsq_multi", &sumsq_multi);
  m.def("ema_multi", &ema_multi);
  m.def("adamw8bit", &adamw8bit);
  m.def("flag_signal", &flag_signal);
  m.def("flag_wait", &flag_wait);
  m.def("flag_barrier", &flag_barrier);
  m.def("rs_finalize", &rs_finalize);
  m.def("rs_adamw", &rs_adamw);
  m.def("peer_gather", &peer_gather);
  m.def("dp_reduce_shard", &dp_reduce_shard);
  m.def("publish_scalar", &publish_scalar);
  m.def("dp_adamw_shard", &dp_adamw_shard);
  m.def("read_status", &read_status);
  m.def("set_wait_limit_ns", &set_wait_limit_ns);
  m.def("attention_set_trace", &attention_set_trace);
}
