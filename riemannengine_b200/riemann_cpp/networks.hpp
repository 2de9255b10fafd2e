// Example networks written against the public layer API of riemann_b200.hpp exactly as a user of the
// reference writes them against its headers (the reference's own examples: tests/train.cpp:629-758 and
// docs/examples.md:171-194 use the same constructor argument lists, ->forward calls, `+` on sparse tensors
// and riemann::cat). They serve two purposes: they show that network code in that style compiles and runs
// unchanged on this host layer, and they are the encoder/decoder the benchmark times.
#pragma once

#include "riemann_b200.hpp"

namespace riemann {
namespace networks {

// convolution -> batch norm -> ReLU
struct ConvNormActImpl : torch::nn::Module {
  RiemannConvolution conv{nullptr};
  RiemannBatchNorm norm{nullptr};
  RiemannReLU act;

  ConvNormActImpl(int c_in, int c_out, int kernel_size = 3, int stride = 1, int dim = 3) {
    conv = register_module("conv", RiemannConvolution(c_in, c_out, kernel_size, stride, /*dilation=*/1, /*bias=*/false,
                                                      /*expand_coordinates=*/false, ConvolutionMode::DEFAULT, dim));
    norm = register_module("norm", RiemannBatchNorm(c_out));
    act = register_module("act", RiemannReLU());
  }
  SparseTensor forward(SparseTensor x) { return act->forward(norm->forward(conv->forward(x))); }
};
TORCH_MODULE(ConvNormAct);

// transposed convolution -> batch norm -> ReLU (the up-sampling step of the decoder)
struct UpNormActImpl : torch::nn::Module {
  RiemannConvolutionTranspose conv{nullptr};
  RiemannBatchNorm norm{nullptr};
  RiemannReLU act;

  UpNormActImpl(int c_in, int c_out, int dim = 3) {
    conv = register_module("conv", RiemannConvolutionTranspose(c_in, c_out, /*kernel_size=*/2, /*stride=*/2, 1, false,
                                                               false, ConvolutionMode::DEFAULT, dim));
    norm = register_module("norm", RiemannBatchNorm(c_out));
    act = register_module("act", RiemannReLU());
  }
  SparseTensor forward(SparseTensor x) { return act->forward(norm->forward(conv->forward(x))); }
};
TORCH_MODULE(UpNormAct);

// Two 3^D convolutions with batch norm, a residual connection and a final ReLU (the reference's BasicBlock,
// engine/nn/residual.cpp:31-52).
struct BasicBlockImpl : torch::nn::Module {
  ConvNormAct first{nullptr};
  RiemannConvolution conv{nullptr};
  RiemannBatchNorm norm{nullptr};
  RiemannReLU act;

  explicit BasicBlockImpl(int channels, int dim = 3) {
    first = register_module("first", ConvNormAct(channels, channels, 3, 1, dim));
    conv = register_module("conv", RiemannConvolution(channels, channels, 3, 1, 1, false, false,
                                                      ConvolutionMode::DEFAULT, dim));
    norm = register_module("norm", RiemannBatchNorm(channels));
    act = register_module("act", RiemannReLU());
  }
  SparseTensor forward(SparseTensor x) {
    auto y = norm->forward(conv->forward(first->forward(x)));
    return act->forward(y + x);
  }
};
TORCH_MODULE(BasicBlock);

// MinkUNet-style encoder/decoder: a 3^D stem, four stages of two BasicBlocks each at widths
// w, 2w, 4w, 8w joined by 2^D stride-2 convolutions, and a decoder of transposed 2^D convolutions whose
// output is concatenated with the encoder features of the same stride and fused by a 3^D convolution.
struct MinkUNetImpl : torch::nn::Module {
  ConvNormAct stem{nullptr};
  std::vector<ConvNormAct> down, fuse;
  std::vector<UpNormAct> up;
  std::vector<BasicBlock> enc_a, enc_b, dec;
  RiemannConvolution head{nullptr};

  MinkUNetImpl(int c_in, int n_out, int width = 32, int dim = 3) {
    stem = register_module("stem", ConvNormAct(c_in, width, 3, 1, dim));
    int c = width;
    for (int s = 0; s < 4; ++s) {
      if (s > 0) {
        down.push_back(register_module("down" + std::to_string(s), ConvNormAct(c, c * 2, 2, 2, dim)));
        c *= 2;
      }
      enc_a.push_back(register_module("enc" + std::to_string(s) + "a", BasicBlock(c, dim)));
      enc_b.push_back(register_module("enc" + std::to_string(s) + "b", BasicBlock(c, dim)));
    }
    for (int s = 3; s > 0; --s) {
      up.push_back(register_module("up" + std::to_string(s), UpNormAct(c, c / 2, dim)));
      fuse.push_back(register_module("fuse" + std::to_string(s), ConvNormAct(c, c / 2, 3, 1, dim)));
      dec.push_back(register_module("dec" + std::to_string(s), BasicBlock(c / 2, dim)));
      c /= 2;
    }
    head = register_module("head", RiemannConvolution(width, n_out, /*kernel_size=*/1, 1, 1, /*bias=*/true, false,
                                                      ConvolutionMode::DEFAULT, dim));
  }

  SparseTensor forward(SparseTensor x) {
    std::vector<SparseTensor> skips;
    auto y = stem->forward(x);
    for (int s = 0; s < 4; ++s) {
      if (s > 0) y = down[s - 1]->forward(y);
      y = enc_b[s]->forward(enc_a[s]->forward(y));
      if (s < 3) skips.push_back(y);
    }
    for (int i = 0; i < 3; ++i) {
      auto u = up[i]->forward(y);
      y = dec[i]->forward(fuse[i]->forward(cat({u, skips[2 - i]})));
    }
    return head->forward(y);
  }
};
TORCH_MODULE(MinkUNet);

}  // namespace networks
}  // namespace riemann
