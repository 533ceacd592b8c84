// Which `a * b + c` sites of the update math are single fma instructions.
//
// PyTorch's CUDA fused optimizers are compiled with nvcc's default -fmad=true, so
// the compiler decided, site by site and template instantiation by template
// instantiation, whether a product feeding a sum became one fma.  Bit-exact
// agreement with `torch.optim.<Opt>(fused=True)` needs the same decisions.  They
// are found empirically: `tests/probe/contraction_search.py` runs every
// combination of the masks in rowmath.cuh against torch._fused_adam_ /
// _fused_adamw_ / _fused_sgd_ / _fused_adagrad_ on the GPU, for every storage type
// and separately for torch's 128-bit vector path and its element-wise path, and
// prints the masks that reproduce torch on every element.
//
// Values below: the result of that search against torch 2.11.0+cu128 on B200
// (1 Mi elements per case; Adam 72 cases, SGD 108 + 18, Adagrad 144 per path and
// storage type).  For fp32 storage the search left exactly one mask for Adam (3),
// SGD with a buffer (29: the momentum blend is fma(1 - dampening, g,
// momentum * buf)) and SGD without (17).  For Adagrad it fixed the accumulator
// site (fused).  The two fp64 sites of Adagrad (weight decay: double(param) *
// double(wd) + double(grad); corrected learning rate: 1 + double(step - 1) *
// double(lr_decay)) cannot be told apart with float math and need not be: every
// operand of those products is an fp32 value widened to fp64, so the product has
// at most 48 significant bits and is exact in fp64; the fused and the unfused form
// then round the same exact sum once and are identical.  They are written fused.
// powf(beta, step) matched torch.pow for 1.8 M arguments.
//
// Fuse<T>::*Vec is used by the 128-bit streaming kernels, *Elem by the element-wise
// kernels (ragged row length, misaligned or strided buffers), mirroring which of
// its two paths torch itself takes for the same layout.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "rowmath.cuh"

namespace cb200 {

constexpr int kSgdFuseAllBuf = kSgdFuseWd | (2 << kSgdBlendShift) | kSgdFuseNesterov | kSgdFuseUpdate;
constexpr int kSgdFuseAllPlain = kSgdFuseWd | kSgdFuseUpdate;

// Default: what fp32 storage showed.  Specialise per storage type where torch's
// instantiation for that type decided differently.
template <class T>
struct Fuse {
  static constexpr int kAdamVec = kAdamFuseAll;
  static constexpr int kAdamElem = kAdamFuseAll;
  static constexpr int kSgdBufVec = kSgdFuseAllBuf;    // torch depth 3
  static constexpr int kSgdBufElem = kSgdFuseAllBuf;
  static constexpr int kSgdPlainVec = kSgdFuseAllPlain;  // torch depth 2
  static constexpr int kSgdPlainElem = kSgdFuseAllPlain;
  static constexpr int kAdagradVec = kAdagradFuseAll;
  static constexpr int kAdagradElem = kAdagradFuseAll;
};

}  // namespace cb200
