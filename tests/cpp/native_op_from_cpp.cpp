// Calls quant_cast_cuda_native::mxfp8 through the PyTorch dispatcher from a C++ program (no Python), and checks the
// result against the C ABI called directly on the same input.  Exit code 0 = same bytes.
#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAStream.h>

#include <cstdio>
#include <string>
#include <vector>

#include "../../include/quant_cast_cuda.h"

int main()
{
    at::manual_seed(0);
    const int64_t M = 256, N = 512;
    at::Tensor x = at::randn({M, N}, at::TensorOptions().device(at::kCUDA).dtype(at::kFloat)).to(at::kBFloat16).contiguous();
    auto op = c10::Dispatcher::singleton()
                  .findSchemaOrThrow("quant_cast_cuda_native::mxfp8", "")
                  .typed<std::vector<at::Tensor>(const at::Tensor &, bool, bool, bool, std::string)>();
    std::vector<at::Tensor> outs = op.call(x, true, true, true, "rceil");
    if (outs.size() != 4) { std::printf("expected four outputs, got %zu\n", outs.size()); return 2; }

    at::Tensor qk = at::empty({M, N}, x.options().dtype(at::kByte)), sk = at::empty({2, 4, 32, 16}, x.options().dtype(at::kByte));
    at::Tensor qm = at::empty({N, M}, x.options().dtype(at::kByte)), sm = at::empty({4, 2, 32, 16}, x.options().dtype(at::kByte));
    int rc = qcc_mxfp8(x.data_ptr(), M, N, QCC_ROWWISE | QCC_COLWISE | QCC_SWIZZLE, qk.data_ptr(), sk.data_ptr(), qm.data_ptr(), sm.data_ptr(),
                       c10::cuda::getCurrentCUDAStream().stream());
    if (rc != 0) { std::printf("qcc_mxfp8 returned %d\n", rc); return 3; }
    const at::Tensor want[4] = {qk, sk, qm, sm};
    for (int i = 0; i < 4; i++) {
        if (!at::equal(outs[i].view(at::kByte), want[i])) { std::printf("output %d differs\n", i); return 1; }
    }
    std::printf("mxfp8 through the dispatcher from C++ equals the C ABI: ok (%lld x %lld)\n", (long long)M, (long long)N);
    return 0;
}
