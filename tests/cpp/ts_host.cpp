// C++ host for a scripted SRU: the boundary test a C++ application of the reference performs
// (sru/csrc/main_test_cpp.cpp + test/test.sh: load a TorchScript module, run it, print h and c with four
// decimals, diff against Python).  This program links libsru_b200_torch.so with --no-as-needed, so the operator
// registrations (sru_cuda::*, sru_b200::*) run when the process loads, before the module is deserialised.
//
//   ts_host <module.pt> [bf16]
//
// The module runs on cuda:0 (this library has no CPU path).  Input: x[t, b, j] = sin(0.37 * (t*B*n + b*n + j)),
// length 5, batch 3, width = the module's input_size; "bf16" converts module and input to bfloat16 first.
#include <torch/script.h>

#include <cmath>
#include <cstring>
#include <iomanip>
#include <iostream>
#include <vector>

int main(int argc, const char *argv[]) {
    if (argc != 2 && argc != 3) {
        std::cerr << "usage: ts_host <scripted-module.pt> [bf16]\n";
        return 2;
    }
    const bool bf16 = argc == 3 && std::strcmp(argv[2], "bf16") == 0;
    torch::NoGradGuard no_grad;
    torch::jit::script::Module module = torch::jit::load(argv[1]);
    module.to(torch::kCUDA);
    if (bf16) module.to(torch::kBFloat16);
    module.eval();
    const int64_t n_in = module.attr("input_size").toInt();
    const int64_t L = 5, B = 3;
    torch::Tensor x = torch::sin(torch::arange(L * B * n_in, torch::kFloat32) * 0.37).view({L, B, n_in}).to(torch::kCUDA);
    if (bf16) x = x.to(torch::kBFloat16);
    std::vector<torch::jit::IValue> inputs{x};
    auto out = module.forward(std::move(inputs)).toTuple();
    for (int which = 0; which < 2; ++which) {
        torch::Tensor t = out->elements()[which].toTensor().to(torch::kFloat32).cpu().contiguous().view({-1});
        const float *p = t.data_ptr<float>();
        for (int64_t i = 0; i < t.numel(); ++i) std::cout << std::fixed << std::setprecision(4) << p[i] << ' ';
        std::cout << std::endl;
    }
    return 0;
}
