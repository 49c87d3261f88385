// Convolution operators of torch.ops.cosmos_b200 (kernels in conv3d_cl.cu): channels-last implicit-GEMM convolution and the
// RMS-norm + SiLU that precedes it in the VAE's residual blocks.

#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <vector>

#include "launchers.h"

int* cb200_error_word(int device);

namespace {
using at::Tensor;

int sm_count(int device) {
  static int counts[64] = {0};
  if (counts[device] == 0) counts[device] = at::cuda::getDeviceProperties(device)->multiProcessorCount;
  return counts[device];
}

// x [T_in, H_in, W_in, Cin] bf16; w [n_rows, ntaps * ceil(Cin / 64) * 64] bf16 (tap-major, channels zero-padded to 64);
// taps: ntaps * 3 ints (dt, dh, dw) added to the output coordinate; out_map: 10 ints (see ConvParams); y is written in place.
void conv_cl(const Tensor& x, const Tensor& w, int64_t n_tile, int64_t Cout, c10::ArrayRef<int64_t> taps, int64_t T_out, int64_t H_out,
             int64_t W_out, c10::ArrayRef<int64_t> out_map, Tensor y, const c10::optional<Tensor>& resid,
             const c10::optional<Tensor>& bias) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 4, "x must be contiguous CUDA bf16 [T, H, W, C]");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.is_contiguous() && w.dim() == 2 && w.device() == x.device(),
              "w must be contiguous CUDA bf16 [rows, K] on the device of x");
  TORCH_CHECK(y.is_cuda() && y.scalar_type() == at::kBFloat16 && y.is_contiguous() && y.device() == x.device(), "y must be contiguous CUDA bf16");
  const int64_t ntaps = (int64_t)taps.size() / 3, Cin = x.size(3), kblocks = (Cin + 63) / 64;
  TORCH_CHECK(taps.size() % 3 == 0 && ntaps >= 1 && ntaps <= 27, "taps: 1..27 triples");
  TORCH_CHECK(out_map.size() == 10, "out_map: 10 integers");
  TORCH_CHECK(Cin % 16 == 0, "input channels must be a multiple of 16");
  TORCH_CHECK(n_tile % 16 == 0 && n_tile >= 16 && n_tile <= 256 && w.size(0) % n_tile == 0 && Cout >= 1 && Cout <= w.size(0), "bad N tiling");
  TORCH_CHECK(w.size(1) == ntaps * kblocks * 64, "weight K extent must be taps * ceil(Cin / 64) * 64");
  TORCH_CHECK(T_out >= 1 && H_out >= 1 && W_out >= 1, "empty output grid");
  // the largest output element the kernel can touch must lie inside y (and inside resid)
  const int64_t ot_mul = out_map[0], ot_add = out_map[1], oh_mul = out_map[2], oh_add = out_map[3], ow_mul = out_map[4], ow_add = out_map[5],
                out_H = out_map[6], out_W = out_map[7], out_C = out_map[8], oc_add = out_map[9];
  TORCH_CHECK(ot_mul >= 1 && oh_mul >= 1 && ow_mul >= 1 && ot_add >= 0 && oh_add >= 0 && ow_add >= 0 && oc_add >= 0, "bad output map");
  TORCH_CHECK((H_out - 1) * oh_mul + oh_add < out_H && (W_out - 1) * ow_mul + ow_add < out_W && oc_add + Cout <= out_C, "output map leaves the frame");
  const int64_t last = ((((T_out - 1) * ot_mul + ot_add) * out_H + out_H - 1) * out_W + out_W - 1) * out_C + out_C;
  TORCH_CHECK(last <= y.numel(), "output map runs past y");
  if (resid.has_value())
    TORCH_CHECK(resid->is_cuda() && resid->scalar_type() == at::kBFloat16 && resid->is_contiguous() && resid->device() == x.device() &&
                    resid->numel() >= last, "resid must be contiguous CUDA bf16 covering the output map");
  if (bias.has_value())
    TORCH_CHECK(bias->is_cuda() && bias->scalar_type() == at::kFloat && bias->is_contiguous() && bias->device() == x.device() &&
                    bias->numel() >= Cout, "bias must be contiguous CUDA fp32 [Cout]");
  c10::cuda::CUDAGuard g(x.device());
  std::vector<int> tp(taps.begin(), taps.end()), om(out_map.begin(), out_map.end());
  const int dev = x.get_device();
  const int rc = cb200_conv_cl(x.data_ptr(), (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)Cin, w.data_ptr(), (int)w.size(0),
                               (int)n_tile, (int)Cout, tp.data(), (int)ntaps, (int)T_out, (int)H_out, (int)W_out, om.data(), y.data_ptr(),
                               resid.has_value() ? resid->data_ptr() : nullptr, bias.has_value() ? bias->data_ptr<float>() : nullptr,
                               cb200_error_word(dev), sm_count(dev), at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "conv_cl launch failed with code ", rc);
}

// y = [silu](x / max(||x||_2, 1e-12) * sqrt(C) * gamma) over the last dimension of a channels-last tensor
Tensor rmsnorm_silu_cl(const Tensor& x, const Tensor& gamma, bool silu) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() >= 2, "x must be contiguous CUDA bf16 [..., C]");
  const int64_t C = x.size(-1);
  TORCH_CHECK(gamma.is_cuda() && gamma.scalar_type() == at::kFloat && gamma.is_contiguous() && gamma.numel() == C && gamma.device() == x.device(),
              "gamma must be contiguous CUDA fp32 [C] on the device of x");
  TORCH_CHECK(C % 8 == 0 && C <= 1024, "channels must be a multiple of 8, at most 1024");
  c10::cuda::CUDAGuard g(x.device());
  Tensor y = at::empty_like(x);
  const int rc = cb200_rmsnorm_silu_cl(x.data_ptr(), gamma.data_ptr<float>(), y.data_ptr(), x.numel() / C, (int)C, silu ? 1 : 0,
                                       at::cuda::getCurrentCUDAStream().stream());
  TORCH_CHECK(rc == 0, "rmsnorm_silu_cl launch failed with code ", rc);
  return y;
}
}  // namespace

void register_conv_ops(torch::Library& m) {
  m.def("conv_cl(Tensor x, Tensor w, int n_tile, int Cout, int[] taps, int T_out, int H_out, int W_out, int[] out_map, Tensor(a!) y, "
        "Tensor? resid, Tensor? bias) -> ()", &conv_cl);
  m.def("rmsnorm_silu_cl(Tensor x, Tensor gamma, bool silu) -> Tensor", &rmsnorm_silu_cl);
}
