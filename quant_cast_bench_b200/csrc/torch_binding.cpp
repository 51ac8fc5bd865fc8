// The casts as native PyTorch operators: TORCH_LIBRARY(quant_cast_cuda_native, ...) over the C ABI.
//
// A thin layer: every operator checks its tensors, allocates the outputs with the gold shapes and dtype views, and
// calls the entry point of include/quant_cast_cuda.h on the current CUDA stream of x's device.  Meta implementations
// give the same shapes without touching a device, so the operators trace (torch.compile, torch.export) and can be
// called from C++ (torch::Dispatcher / the generated torch.ops handles) without Python.  The reference's counterpart is
// the recipe layer of its Triton backend (quant_cast_triton/recipes.py:48-65 of vkuzo/quant_cast_bench).
//
//   amax(x, kind, fmt, recip_div)                           -> fp32 scalar   kind: "raw" | "fp8" | "nvfp4"
//   fp8_tensorwise(x, scale, fmt)                           -> q
//   fp8_rowwise(x, fmt, recip_div)                          -> (q, scale (M, 1))
//   fp8_colwise(x, fmt, recip_div)                          -> (q (N, M), scale (N, 1))
//   mxfp8(x, rowwise, colwise, swizzle, mode)               -> [qk, sk][qm, sm]   mode: "rceil" | "floor"
//   nvfp4(x, outer_scale, swizzle, transposed, recip_div)   -> (q, inner scales)   outer_scale: one value, (M, 1) per
//                                                               token, or the (M/128, N/128) grid of 128x128 blocks
//   nvfp4_sr(x, outer_scale, key, swizzle, transposed, recip_div) -> (q, inner scales)   key: uint64 [seed, offset]
//   nvfp4_both(x, outer_scale, swizzle, recip_div)          -> (qk, sk, qm, sm)     both orientations from one read
//   fp8_rowwise_precalc(x, scale, fmt) / fp8_colwise_precalc(x, scale, fmt) -> q   true division by given scales
//   fp8_block128(x, rowwise, colwise, recip_div)            -> [qk, sk][qm, sm]    1x128 / 128x1 blocks, fp32 scales
//   fp8_block128x128(x, recip_div)                          -> (q, scale (M/128, N/128))
//   mxfp8_32x32(x, rowwise, colwise, swizzle, transposed_data) -> [qk, sk][qm] [sm] one e8m0 scale per 32x32 block
//   mxfp4(x, swizzle)                                       -> (q (M, N/2), scale)
//   nvfp4_per_token_scale(x, recip_div)                     -> (M, 1) fp32 outer scales
//   sr_f32_to_bf16(x, key, global_row, global_col, num_col) -> bf16       fp32 input, stochastic rounding
//
// recip_div: QCC_RECIP_DIV (divisions by a constant as eager PyTorch computes them on a CUDA device).
// Built by quant_cast_bench_b200/build.py into lib/libquant_cast_torch.so, which links against libquant_cast_cuda.so.
#include <ATen/ATen.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/library.h>

#include <string>
#include <tuple>
#include <vector>

#include "../../include/quant_cast_cuda.h"

namespace {

void check_x(const at::Tensor &x)
{
    TORCH_CHECK(x.dim() == 2, "quant_cast_cuda: x must be 2-D");
    TORCH_CHECK(x.scalar_type() == at::kBFloat16, "quant_cast_cuda: x must be bfloat16");
}
void check_x_cuda(const at::Tensor &x)
{
    check_x(x);
    TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "quant_cast_cuda: x must be a contiguous CUDA tensor (there is no CPU implementation)");
}
// an auxiliary tensor (scale, key) must live on x's device: the kernels read it there
void same_device(const at::Tensor &x, const at::Tensor &aux, const char *what)
{
    TORCH_CHECK(aux.device() == x.device(), "quant_cast_cuda: ", what, " is on ", aux.device(), ", x on ", x.device());
}
void *stream_of(const at::Tensor &x) { return c10::cuda::getCurrentCUDAStream(x.get_device()).stream(); }
void ok(int rc, const char *what) { TORCH_CHECK(rc == 0, "quant_cast_cuda: ", what, " failed with code ", rc); }
int fmt_of(const std::string &fmt)
{
    TORCH_CHECK(fmt == "e4m3" || fmt == "e5m2", "quant_cast_cuda: fmt must be 'e4m3' or 'e5m2'");
    return fmt == "e5m2" ? QCC_FMT_E5M2 : QCC_FMT_E4M3;
}
at::ScalarType fp8_dtype(const std::string &fmt) { return fmt_of(fmt) == QCC_FMT_E5M2 ? at::kFloat8_e5m2 : at::kFloat8_e4m3fn; }
int amax_mode(const std::string &kind)
{
    TORCH_CHECK(kind == "raw" || kind == "fp8" || kind == "nvfp4", "quant_cast_cuda: kind must be 'raw', 'fp8' or 'nvfp4'");
    return kind == "raw" ? QCC_AMAX_RAW : kind == "fp8" ? QCC_AMAX_FP8_SCALE : QCC_AMAX_NVFP4_SCALE;
}
int mx_mode(const std::string &mode)
{
    TORCH_CHECK(mode == "rceil" || mode == "floor", "quant_cast_cuda: mode must be 'rceil' or 'floor'");
    return mode == "floor" ? QCC_FLOOR : 0;
}
std::vector<int64_t> blocked_shape(int64_t rows, int64_t cols) { return {(rows + 127) / 128, (cols + 3) / 4, 32, 16}; }
std::vector<int64_t> scale_shape(int64_t rows, int64_t cols, bool swizzle)
{
    return swizzle ? blocked_shape(rows, cols) : std::vector<int64_t>{rows, cols};
}
at::Tensor bytes(at::IntArrayRef shape, const at::Tensor &like) { return at::empty(shape, like.options().dtype(at::kByte)); }

// ---------------------------------------------------------------------------------------- CUDA implementations
at::Tensor amax_cuda(const at::Tensor &x, std::string kind, std::string fmt, bool recip_div)
{
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "quant_cast_cuda: x must be contiguous CUDA bfloat16");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor out = at::empty({}, x.options().dtype(at::kFloat));
    const size_t ws_bytes = qcc_amax_workspace_bytes();
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));   // two launches: any contents will do
    ok(qcc_amax_bf16(x.data_ptr(), x.numel(), amax_mode(kind) | (recip_div ? QCC_RECIP_DIV : 0), fmt_of(fmt), out.data_ptr<float>(),
                     ws.data_ptr(), ws_bytes, stream_of(x)),
       "amax");
    return out;
}

at::Tensor fp8_tensorwise_cuda(const at::Tensor &x, const at::Tensor &scale, std::string fmt)
{
    check_x_cuda(x);
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == 1, "quant_cast_cuda: scale must be one CUDA fp32 value");
    same_device(x, scale, "scale");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor q = bytes(x.sizes(), x);
    ok(qcc_fp8_tensorwise(x.data_ptr(), x.numel(), scale.data_ptr<float>(), fmt_of(fmt), q.data_ptr(), stream_of(x)), "fp8_tensorwise");
    return q.view(fp8_dtype(fmt));
}

std::tuple<at::Tensor, at::Tensor> fp8_rowwise_cuda(const at::Tensor &x, std::string fmt, bool recip_div)
{
    check_x_cuda(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    at::Tensor q = bytes({M, N}, x), s = at::empty({M, 1}, x.options().dtype(at::kFloat));
    ok(qcc_fp8_rowwise(x.data_ptr(), M, N, fmt_of(fmt) | (recip_div ? QCC_RECIP_DIV : 0), q.data_ptr(), s.data_ptr<float>(), stream_of(x)),
       "fp8_rowwise");
    return {q.view(fp8_dtype(fmt)), s};
}

std::tuple<at::Tensor, at::Tensor> fp8_colwise_cuda(const at::Tensor &x, std::string fmt, bool recip_div)
{
    check_x_cuda(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(M % 16 == 0 && N % 8 == 0, "quant_cast_cuda: colwise fp8 needs M % 16 == 0 and N % 8 == 0");
    at::Tensor q = bytes({N, M}, x), s = at::empty({N, 1}, x.options().dtype(at::kFloat));
    const size_t ws_bytes = qcc_fp8_colwise_workspace_bytes(M, N);
    at::Tensor ws = at::empty({(int64_t)ws_bytes}, x.options().dtype(at::kByte));
    ok(qcc_fp8_colwise(x.data_ptr(), M, N, fmt_of(fmt) | (recip_div ? QCC_RECIP_DIV : 0), q.data_ptr(), s.data_ptr<float>(), ws.data_ptr(),
                       ws_bytes, stream_of(x)),
       "fp8_colwise");
    return {q.view(fp8_dtype(fmt)), s};
}

std::vector<at::Tensor> mxfp8_cuda(const at::Tensor &x, bool rowwise, bool colwise, bool swizzle, std::string mode)
{
    check_x_cuda(x);
    TORCH_CHECK(rowwise || colwise, "quant_cast_cuda: mxfp8 needs at least one direction");
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK((!rowwise || N % 32 == 0) && (!colwise || (M % 32 == 0 && N % 8 == 0)), "quant_cast_cuda: mxfp8 blocks need N % 32 == 0 (rowwise) / M % 32 == 0 (colwise)");
    at::Tensor qk, sk, qm, sm;
    if (rowwise) { qk = bytes({M, N}, x); sk = bytes(scale_shape(M, N / 32, swizzle), x); }
    if (colwise) { qm = bytes({N, M}, x); sm = bytes(scale_shape(N, M / 32, swizzle), x); }
    const int flags = (rowwise ? QCC_ROWWISE : 0) | (colwise ? QCC_COLWISE : 0) | (swizzle ? QCC_SWIZZLE : 0) | mx_mode(mode);
    ok(qcc_mxfp8(x.data_ptr(), M, N, flags, rowwise ? qk.data_ptr() : nullptr, rowwise ? sk.data_ptr() : nullptr,
                 colwise ? qm.data_ptr() : nullptr, colwise ? sm.data_ptr() : nullptr, stream_of(x)),
       "mxfp8");
    std::vector<at::Tensor> outs;
    if (rowwise) { outs.push_back(qk.view(at::kFloat8_e4m3fn)); outs.push_back(sk.view(at::kFloat8_e8m0fnu)); }
    if (colwise) { outs.push_back(qm.view(at::kFloat8_e4m3fn)); outs.push_back(sm.view(at::kFloat8_e8m0fnu)); }
    return outs;
}

// which outer scale: 0 one value, 1 one per row (M, 1), 2 one per 128x128 block (M/128, N/128)
int outer_kind(const at::Tensor &x, const at::Tensor &outer)
{
    const int64_t M = x.size(0), N = x.size(1);
    if (outer.numel() == 1 && outer.dim() < 2) return 0;
    if (outer.dim() == 2 && outer.size(0) == M && outer.size(1) == 1) return 1;
    if (outer.dim() == 2 && M % 128 == 0 && N % 128 == 0 && outer.size(0) == M / 128 && outer.size(1) == N / 128) return 2;
    if (outer.numel() == 1) return 0;
    TORCH_CHECK(false, "quant_cast_cuda: outer_scale must be one value, (M, 1), or (M/128, N/128)");
    return -1;
}

std::tuple<at::Tensor, at::Tensor> nvfp4_impl(const at::Tensor &x, const at::Tensor &outer_in, const uint64_t *key, bool swizzle,
                                              bool transposed, bool recip_div)
{
    check_x_cuda(x);
    TORCH_CHECK(outer_in.is_cuda() && outer_in.scalar_type() == at::kFloat, "quant_cast_cuda: outer_scale must be a CUDA fp32 tensor");
    same_device(x, outer_in, "outer_scale");
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    const at::Tensor outer = outer_in.contiguous();
    const int kind = outer_kind(x, outer);
    const int flags = (swizzle ? QCC_SWIZZLE : 0) | (recip_div ? QCC_RECIP_DIV : 0) | (key ? QCC_SR : 0);
    at::Tensor q, s;
    if (transposed) {
        TORCH_CHECK(kind == 0, "quant_cast_cuda: the transposed nvfp4 cast takes one outer scale");
        TORCH_CHECK(M % 32 == 0 && N % 8 == 0, "quant_cast_cuda: transposed nvfp4 needs M % 32 == 0 and N % 8 == 0");
        q = bytes({N, M / 2}, x);
        s = bytes(scale_shape(N, M / 16, swizzle), x);
        ok(qcc_nvfp4_transposed(x.data_ptr(), M, N, outer.data_ptr<float>(), flags, key, q.data_ptr(), s.data_ptr(), stream_of(x)),
           "nvfp4 transposed");
    } else {
        TORCH_CHECK(N % 16 == 0, "quant_cast_cuda: nvfp4 needs N % 16 == 0");
        TORCH_CHECK(kind != 2 || (swizzle && !key), "quant_cast_cuda: a blocked outer scale goes with blocked inner scales and round to nearest");
        q = bytes({M, N / 2}, x);
        s = bytes(scale_shape(M, N / 16, swizzle), x);
        ok(qcc_nvfp4(x.data_ptr(), M, N, outer.data_ptr<float>(), kind, flags, key, q.data_ptr(), s.data_ptr(), stream_of(x)), "nvfp4");
    }
    return {q.view(at::kFloat4_e2m1fn_x2), s.view(at::kFloat8_e4m3fn)};
}

std::tuple<at::Tensor, at::Tensor> nvfp4_cuda(const at::Tensor &x, const at::Tensor &outer_scale, bool swizzle, bool transposed,
                                              bool recip_div)
{
    return nvfp4_impl(x, outer_scale, nullptr, swizzle, transposed, recip_div);
}

std::tuple<at::Tensor, at::Tensor> nvfp4_sr_cuda(const at::Tensor &x, const at::Tensor &outer_scale, const at::Tensor &key, bool swizzle,
                                                 bool transposed, bool recip_div)
{
    TORCH_CHECK(key.is_cuda() && key.element_size() == 8 && key.numel() >= 2 && key.is_contiguous(),
                "quant_cast_cuda: key must be a CUDA tensor of two 64-bit words [seed, offset]");
    same_device(x, key, "key");
    return nvfp4_impl(x, outer_scale, static_cast<const uint64_t *>(key.data_ptr()), swizzle, transposed, recip_div);
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> nvfp4_both_cuda(const at::Tensor &x, const at::Tensor &outer_scale, bool swizzle,
                                                                         bool recip_div)
{
    check_x_cuda(x);
    TORCH_CHECK(outer_scale.is_cuda() && outer_scale.scalar_type() == at::kFloat && outer_scale.numel() == 1,
                "quant_cast_cuda: outer_scale must be one CUDA fp32 value");
    same_device(x, outer_scale, "outer_scale");
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(M % 32 == 0 && N % 32 == 0, "quant_cast_cuda: nvfp4 in both orientations needs M % 32 == 0 and N % 32 == 0");
    at::Tensor qk = bytes({M, N / 2}, x), sk = bytes(scale_shape(M, N / 16, swizzle), x);
    at::Tensor qm = bytes({N, M / 2}, x), sm = bytes(scale_shape(N, M / 16, swizzle), x);
    ok(qcc_nvfp4_both(x.data_ptr(), M, N, outer_scale.data_ptr<float>(), (swizzle ? QCC_SWIZZLE : 0) | (recip_div ? QCC_RECIP_DIV : 0),
                      qk.data_ptr(), sk.data_ptr(), qm.data_ptr(), sm.data_ptr(), stream_of(x)),
       "nvfp4 both");
    return {qk.view(at::kFloat4_e2m1fn_x2), sk.view(at::kFloat8_e4m3fn), qm.view(at::kFloat4_e2m1fn_x2), sm.view(at::kFloat8_e4m3fn)};
}

at::Tensor fp8_rowwise_precalc_cuda(const at::Tensor &x, const at::Tensor &scale, std::string fmt)
{
    check_x_cuda(x);
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == M, "quant_cast_cuda: scale must hold one CUDA fp32 value per row");
    same_device(x, scale, "scale");
    const c10::cuda::CUDAGuard guard(x.device());
    const at::Tensor sc = scale.contiguous();
    at::Tensor q = bytes({M, N}, x);
    ok(qcc_fp8_rowwise_precalc(x.data_ptr(), M, N, sc.data_ptr<float>(), fmt_of(fmt), q.data_ptr(), stream_of(x)), "fp8_rowwise_precalc");
    return q.view(fp8_dtype(fmt));
}

at::Tensor fp8_colwise_precalc_cuda(const at::Tensor &x, const at::Tensor &scale, std::string fmt)
{
    check_x_cuda(x);
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(scale.is_cuda() && scale.scalar_type() == at::kFloat && scale.numel() == N, "quant_cast_cuda: scale must hold one CUDA fp32 value per column");
    same_device(x, scale, "scale");
    TORCH_CHECK(M % 16 == 0 && N % 8 == 0, "quant_cast_cuda: colwise fp8 needs M % 16 == 0 and N % 8 == 0");
    const c10::cuda::CUDAGuard guard(x.device());
    const at::Tensor sc = scale.contiguous();
    at::Tensor q = bytes({N, M}, x);
    ok(qcc_fp8_colwise_precalc(x.data_ptr(), M, N, sc.data_ptr<float>(), fmt_of(fmt), q.data_ptr(), stream_of(x)), "fp8_colwise_precalc");
    return q.view(fp8_dtype(fmt));
}

std::vector<at::Tensor> fp8_block128_cuda(const at::Tensor &x, bool rowwise, bool colwise, bool recip_div)
{
    check_x_cuda(x);
    TORCH_CHECK(rowwise || colwise, "quant_cast_cuda: fp8_block128 needs at least one direction");
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK((!rowwise || N % 128 == 0) && (!colwise || (M % 128 == 0 && N % 8 == 0)),
                "quant_cast_cuda: 1x128 blocks need N % 128 == 0, 128x1 blocks M % 128 == 0 and N % 8 == 0");
    at::Tensor qk, sk, qm, sm;
    if (rowwise) { qk = bytes({M, N}, x); sk = at::empty({M, N / 128}, x.options().dtype(at::kFloat)); }
    if (colwise) { qm = bytes({N, M}, x); sm = at::empty({N, M / 128}, x.options().dtype(at::kFloat)); }
    const int flags = (rowwise ? QCC_ROWWISE : 0) | (colwise ? QCC_COLWISE : 0) | (recip_div ? QCC_RECIP_DIV : 0);
    ok(qcc_fp8_block128(x.data_ptr(), M, N, flags, rowwise ? qk.data_ptr() : nullptr, rowwise ? sk.data_ptr<float>() : nullptr,
                        colwise ? qm.data_ptr() : nullptr, colwise ? sm.data_ptr<float>() : nullptr, stream_of(x)),
       "fp8_block128");
    std::vector<at::Tensor> outs;
    if (rowwise) { outs.push_back(qk.view(at::kFloat8_e4m3fn)); outs.push_back(sk); }
    if (colwise) { outs.push_back(qm.view(at::kFloat8_e4m3fn)); outs.push_back(sm); }
    return outs;
}

std::tuple<at::Tensor, at::Tensor> fp8_block128x128_cuda(const at::Tensor &x, bool recip_div)
{
    check_x_cuda(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(M % 128 == 0 && N % 128 == 0, "quant_cast_cuda: 128x128 blocks need M % 128 == 0 and N % 128 == 0");
    at::Tensor q = bytes({M, N}, x), s = at::empty({M / 128, N / 128}, x.options().dtype(at::kFloat));
    ok(qcc_fp8_block128x128(x.data_ptr(), M, N, recip_div ? QCC_RECIP_DIV : 0, q.data_ptr(), s.data_ptr<float>(), stream_of(x)), "fp8_block128x128");
    return {q.view(at::kFloat8_e4m3fn), s};
}

std::vector<at::Tensor> mxfp8_32x32_cuda(const at::Tensor &x, bool rowwise, bool colwise, bool swizzle, bool transposed_data)
{
    check_x_cuda(x);
    TORCH_CHECK(rowwise || colwise, "quant_cast_cuda: mxfp8_32x32 needs at least one direction");
    TORCH_CHECK(!colwise || swizzle, "quant_cast_cuda: the transposed 32x32 outputs come with blocked scales only");
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(M % 32 == 0 && N % 32 == 0, "quant_cast_cuda: 32x32 blocks need M % 32 == 0 and N % 32 == 0");
    at::Tensor qk, sk, qm, sm;
    if (rowwise) { qk = bytes({M, N}, x); sk = swizzle ? bytes(blocked_shape(M, N / 32), x) : bytes({M / 32, N / 32}, x); }
    if (colwise) { if (transposed_data) qm = bytes({N, M}, x); sm = bytes(blocked_shape(N, M / 32), x); }
    const int flags = QCC_BLOCK32 | (rowwise ? QCC_ROWWISE : 0) | (colwise ? QCC_COLWISE : 0) | (swizzle ? QCC_SWIZZLE : 0);
    ok(qcc_mxfp8(x.data_ptr(), M, N, flags, rowwise ? qk.data_ptr() : nullptr, rowwise ? sk.data_ptr() : nullptr,
                 qm.defined() ? qm.data_ptr() : nullptr, colwise ? sm.data_ptr() : nullptr, stream_of(x)),
       "mxfp8 32x32");
    std::vector<at::Tensor> outs;
    if (rowwise) { outs.push_back(qk.view(at::kFloat8_e4m3fn)); outs.push_back(sk.view(at::kFloat8_e8m0fnu)); }
    if (colwise) { if (transposed_data) outs.push_back(qm.view(at::kFloat8_e4m3fn)); outs.push_back(sm.view(at::kFloat8_e8m0fnu)); }
    return outs;
}

std::tuple<at::Tensor, at::Tensor> mxfp4_cuda(const at::Tensor &x, bool swizzle)
{
    check_x_cuda(x);
    const c10::cuda::CUDAGuard guard(x.device());
    const int64_t M = x.size(0), N = x.size(1);
    TORCH_CHECK(N % 32 == 0, "quant_cast_cuda: mxfp4 needs N % 32 == 0");
    at::Tensor q = bytes({M, N / 2}, x), s = bytes(scale_shape(M, N / 32, swizzle), x);
    ok(qcc_mxfp4(x.data_ptr(), M, N, swizzle ? QCC_SWIZZLE : 0, q.data_ptr(), s.data_ptr(), stream_of(x)), "mxfp4");
    return {q.view(at::kFloat4_e2m1fn_x2), s.view(at::kFloat8_e8m0fnu)};
}

at::Tensor nvfp4_per_token_scale_cuda(const at::Tensor &x, bool recip_div)
{
    check_x_cuda(x);
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor s = at::empty({x.size(0), 1}, x.options().dtype(at::kFloat));
    ok(qcc_nvfp4_per_token_scale(x.data_ptr(), x.size(0), x.size(1), recip_div ? QCC_RECIP_DIV : 0, s.data_ptr<float>(), stream_of(x)),
       "nvfp4_per_token_scale");
    return s;
}

at::Tensor sr_f32_to_bf16_cuda(const at::Tensor &x, const at::Tensor &key, int64_t global_row, int64_t global_col, int64_t num_col)
{
    TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.dim() == 2 && x.scalar_type() == at::kFloat,
                "quant_cast_cuda: sr_f32_to_bf16 takes a contiguous 2-D CUDA fp32 tensor");
    TORCH_CHECK(key.is_cuda() && key.element_size() == 8 && key.numel() >= 2 && key.is_contiguous(),
                "quant_cast_cuda: key must be a CUDA tensor of two 64-bit words [seed, offset]");
    same_device(x, key, "key");
    const c10::cuda::CUDAGuard guard(x.device());
    at::Tensor out = at::empty(x.sizes(), x.options().dtype(at::kBFloat16));
    ok(qcc_sr_f32_to_bf16(x.data_ptr(), x.size(0), x.size(1), static_cast<const uint64_t *>(key.data_ptr()), global_row, global_col,
                          num_col < 0 ? x.size(1) : num_col, out.data_ptr(), stream_of(x)),
       "sr_f32_to_bf16");
    return out;
}

// ---------------------------------------------------------------------------------------- Meta (shape) implementations
at::Tensor like(const at::Tensor &x, std::vector<int64_t> shape, at::ScalarType dt) { return at::empty(shape, x.options().dtype(dt)); }

at::Tensor amax_meta(const at::Tensor &x, std::string kind, std::string fmt, bool)
{
    amax_mode(kind);
    fmt_of(fmt);
    return like(x, {}, at::kFloat);
}
at::Tensor fp8_tensorwise_meta(const at::Tensor &x, const at::Tensor &, std::string fmt) { return like(x, x.sizes().vec(), fp8_dtype(fmt)); }
std::tuple<at::Tensor, at::Tensor> fp8_rowwise_meta(const at::Tensor &x, std::string fmt, bool)
{
    check_x(x);
    return {like(x, {x.size(0), x.size(1)}, fp8_dtype(fmt)), like(x, {x.size(0), 1}, at::kFloat)};
}
std::tuple<at::Tensor, at::Tensor> fp8_colwise_meta(const at::Tensor &x, std::string fmt, bool)
{
    check_x(x);
    return {like(x, {x.size(1), x.size(0)}, fp8_dtype(fmt)), like(x, {x.size(1), 1}, at::kFloat)};
}
std::vector<at::Tensor> mxfp8_meta(const at::Tensor &x, bool rowwise, bool colwise, bool swizzle, std::string mode)
{
    check_x(x);
    mx_mode(mode);
    const int64_t M = x.size(0), N = x.size(1);
    std::vector<at::Tensor> outs;
    if (rowwise) { outs.push_back(like(x, {M, N}, at::kFloat8_e4m3fn)); outs.push_back(like(x, scale_shape(M, N / 32, swizzle), at::kFloat8_e8m0fnu)); }
    if (colwise) { outs.push_back(like(x, {N, M}, at::kFloat8_e4m3fn)); outs.push_back(like(x, scale_shape(N, M / 32, swizzle), at::kFloat8_e8m0fnu)); }
    return outs;
}
std::tuple<at::Tensor, at::Tensor> nvfp4_meta(const at::Tensor &x, const at::Tensor &, bool swizzle, bool transposed, bool)
{
    check_x(x);
    const int64_t rows = transposed ? x.size(1) : x.size(0), cols = transposed ? x.size(0) : x.size(1);
    return {like(x, {rows, cols / 2}, at::kFloat4_e2m1fn_x2), like(x, scale_shape(rows, cols / 16, swizzle), at::kFloat8_e4m3fn)};
}

std::tuple<at::Tensor, at::Tensor> nvfp4_sr_meta(const at::Tensor &x, const at::Tensor &o, const at::Tensor &, bool swizzle, bool transposed,
                                                 bool r)
{
    return nvfp4_meta(x, o, swizzle, transposed, r);
}
std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor> nvfp4_both_meta(const at::Tensor &x, const at::Tensor &, bool swizzle, bool)
{
    check_x(x);
    const int64_t M = x.size(0), N = x.size(1);
    return {like(x, {M, N / 2}, at::kFloat4_e2m1fn_x2), like(x, scale_shape(M, N / 16, swizzle), at::kFloat8_e4m3fn),
            like(x, {N, M / 2}, at::kFloat4_e2m1fn_x2), like(x, scale_shape(N, M / 16, swizzle), at::kFloat8_e4m3fn)};
}
at::Tensor fp8_rowwise_precalc_meta(const at::Tensor &x, const at::Tensor &, std::string fmt)
{
    check_x(x);
    return like(x, {x.size(0), x.size(1)}, fp8_dtype(fmt));
}
at::Tensor fp8_colwise_precalc_meta(const at::Tensor &x, const at::Tensor &, std::string fmt)
{
    check_x(x);
    return like(x, {x.size(1), x.size(0)}, fp8_dtype(fmt));
}
std::vector<at::Tensor> fp8_block128_meta(const at::Tensor &x, bool rowwise, bool colwise, bool)
{
    check_x(x);
    const int64_t M = x.size(0), N = x.size(1);
    std::vector<at::Tensor> outs;
    if (rowwise) { outs.push_back(like(x, {M, N}, at::kFloat8_e4m3fn)); outs.push_back(like(x, {M, N / 128}, at::kFloat)); }
    if (colwise) { outs.push_back(like(x, {N, M}, at::kFloat8_e4m3fn)); outs.push_back(like(x, {N, M / 128}, at::kFloat)); }
    return outs;
}
std::tuple<at::Tensor, at::Tensor> fp8_block128x128_meta(const at::Tensor &x, bool)
{
    check_x(x);
    return {like(x, {x.size(0), x.size(1)}, at::kFloat8_e4m3fn), like(x, {x.size(0) / 128, x.size(1) / 128}, at::kFloat)};
}
std::vector<at::Tensor> mxfp8_32x32_meta(const at::Tensor &x, bool rowwise, bool colwise, bool swizzle, bool transposed_data)
{
    check_x(x);
    const int64_t M = x.size(0), N = x.size(1);
    std::vector<at::Tensor> outs;
    if (rowwise) {
        outs.push_back(like(x, {M, N}, at::kFloat8_e4m3fn));
        outs.push_back(like(x, swizzle ? blocked_shape(M, N / 32) : std::vector<int64_t>{M / 32, N / 32}, at::kFloat8_e8m0fnu));
    }
    if (colwise) {
        if (transposed_data) outs.push_back(like(x, {N, M}, at::kFloat8_e4m3fn));
        outs.push_back(like(x, blocked_shape(N, M / 32), at::kFloat8_e8m0fnu));
    }
    return outs;
}
std::tuple<at::Tensor, at::Tensor> mxfp4_meta(const at::Tensor &x, bool swizzle)
{
    check_x(x);
    return {like(x, {x.size(0), x.size(1) / 2}, at::kFloat4_e2m1fn_x2), like(x, scale_shape(x.size(0), x.size(1) / 32, swizzle), at::kFloat8_e8m0fnu)};
}

at::Tensor nvfp4_per_token_scale_meta(const at::Tensor &x, bool)
{
    check_x(x);
    return like(x, {x.size(0), 1}, at::kFloat);
}
at::Tensor sr_f32_to_bf16_meta(const at::Tensor &x, const at::Tensor &, int64_t, int64_t, int64_t)
{
    TORCH_CHECK(x.dim() == 2 && x.scalar_type() == at::kFloat, "quant_cast_cuda: sr_f32_to_bf16 takes a 2-D fp32 tensor");
    return like(x, x.sizes().vec(), at::kBFloat16);
}

}  // namespace

TORCH_LIBRARY(quant_cast_cuda_native, m)
{
    m.def("amax(Tensor x, str kind, str fmt, bool recip_div=False) -> Tensor");
    m.def("fp8_tensorwise(Tensor x, Tensor scale, str fmt) -> Tensor");
    m.def("fp8_rowwise(Tensor x, str fmt, bool recip_div=False) -> (Tensor, Tensor)");
    m.def("fp8_colwise(Tensor x, str fmt, bool recip_div=False) -> (Tensor, Tensor)");
    m.def("mxfp8(Tensor x, bool rowwise, bool colwise, bool swizzle, str mode) -> Tensor[]");
    m.def("nvfp4(Tensor x, Tensor outer_scale, bool swizzle, bool transposed, bool recip_div=False) -> (Tensor, Tensor)");
    m.def("nvfp4_sr(Tensor x, Tensor outer_scale, Tensor key, bool swizzle, bool transposed, bool recip_div=False) -> (Tensor, Tensor)");
    m.def("nvfp4_both(Tensor x, Tensor outer_scale, bool swizzle, bool recip_div=False) -> (Tensor, Tensor, Tensor, Tensor)");
    m.def("fp8_rowwise_precalc(Tensor x, Tensor scale, str fmt) -> Tensor");
    m.def("fp8_colwise_precalc(Tensor x, Tensor scale, str fmt) -> Tensor");
    m.def("fp8_block128(Tensor x, bool rowwise, bool colwise, bool recip_div=False) -> Tensor[]");
    m.def("fp8_block128x128(Tensor x, bool recip_div=False) -> (Tensor, Tensor)");
    m.def("mxfp8_32x32(Tensor x, bool rowwise, bool colwise, bool swizzle, bool transposed_data=True) -> Tensor[]");
    m.def("mxfp4(Tensor x, bool swizzle) -> (Tensor, Tensor)");
    m.def("nvfp4_per_token_scale(Tensor x, bool recip_div=False) -> Tensor");
    m.def("sr_f32_to_bf16(Tensor x, Tensor key, int global_row=0, int global_col=0, int num_col=-1) -> Tensor");
}

TORCH_LIBRARY_IMPL(quant_cast_cuda_native, CUDA, m)
{
    m.impl("amax", amax_cuda);
    m.impl("fp8_tensorwise", fp8_tensorwise_cuda);
    m.impl("fp8_rowwise", fp8_rowwise_cuda);
    m.impl("fp8_colwise", fp8_colwise_cuda);
    m.impl("mxfp8", mxfp8_cuda);
    m.impl("nvfp4", nvfp4_cuda);
    m.impl("nvfp4_sr", nvfp4_sr_cuda);
    m.impl("nvfp4_both", nvfp4_both_cuda);
    m.impl("fp8_rowwise_precalc", fp8_rowwise_precalc_cuda);
    m.impl("fp8_colwise_precalc", fp8_colwise_precalc_cuda);
    m.impl("fp8_block128", fp8_block128_cuda);
    m.impl("fp8_block128x128", fp8_block128x128_cuda);
    m.impl("mxfp8_32x32", mxfp8_32x32_cuda);
    m.impl("mxfp4", mxfp4_cuda);
    m.impl("nvfp4_per_token_scale", nvfp4_per_token_scale_cuda);
    m.impl("sr_f32_to_bf16", sr_f32_to_bf16_cuda);
}

TORCH_LIBRARY_IMPL(quant_cast_cuda_native, Meta, m)
{
    m.impl("amax", amax_meta);
    m.impl("fp8_tensorwise", fp8_tensorwise_meta);
    m.impl("fp8_rowwise", fp8_rowwise_meta);
    m.impl("fp8_colwise", fp8_colwise_meta);
    m.impl("mxfp8", mxfp8_meta);
    m.impl("nvfp4", nvfp4_meta);
    m.impl("nvfp4_sr", nvfp4_sr_meta);
    m.impl("nvfp4_both", nvfp4_both_meta);
    m.impl("fp8_rowwise_precalc", fp8_rowwise_precalc_meta);
    m.impl("fp8_colwise_precalc", fp8_colwise_precalc_meta);
    m.impl("fp8_block128", fp8_block128_meta);
    m.impl("fp8_block128x128", fp8_block128x128_meta);
    m.impl("mxfp8_32x32", mxfp8_32x32_meta);
    m.impl("mxfp4", mxfp4_meta);
    m.impl("nvfp4_per_token_scale", nvfp4_per_token_scale_meta);
    m.impl("sr_f32_to_bf16", sr_f32_to_bf16_meta);
}
