// Thread mapping shared by the token-by-token forward and backward kernels: a CTA
// keeps a D x D fp32 matrix in registers, thread (kq, vq) owning rows
// [kq*R, kq*R + R) and the four columns [4 vq, 4 vq + 4).
#pragma once

namespace pkda {

template <int D> struct RecCfg {
  static constexpr int kThreads = D >= 32 ? 256 : (D == 16 ? 64 : 32);
  static constexpr int kVQ = D / 4;                                        // threads across v
  static constexpr int kKW = (kThreads / kVQ) < D ? (kThreads / kVQ) : D;  // row groups
  static constexpr int kActive = kVQ * kKW;
  static constexpr int kR = D / kKW;                                       // rows per thread
};

}  // namespace pkda
