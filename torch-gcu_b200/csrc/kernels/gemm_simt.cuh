// Exact-order SIMT matrix multiply: the path for fp32 / fp64 operands (whose
// results the reference's unit tests pin against CPU fp32 arithmetic) and for
// any layout the tensor-core kernel does not take. 64x64 output tile per block,
// 16x16 threads with a 4x4 micro-tile each, K stepped 16 at a time through
// shared memory; operands are addressed through their element strides, so every
// transposition / batch broadcast works.
#pragma once

#include "common.cuh"

namespace b200 {
namespace simt {

struct MatmulArgs {
  const void* a; const void* b; const void* cin; void* out;
  int64_t M, N, K, batch;
  int64_t a_sb, a_sm, a_sk;
  int64_t b_sb, b_sk, b_sn;
  int64_t c_sb, c_sm, c_sn;   // cin strides (0 = broadcast)
  int64_t o_sb, o_sm, o_sn;
  double alpha, beta;
};

template <typename T, typename Acc>
__global__ void __launch_bounds__(256)
matmul_kernel(MatmulArgs p) {
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ Acc As[BK][BM + 1];
  __shared__ Acc Bs[BK][BN + 1];
  const int64_t batch = blockIdx.z;
  const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
  const T* A = static_cast<const T*>(p.a) + batch * p.a_sb;
  const T* B = static_cast<const T*>(p.b) + batch * p.b_sb;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  Acc acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = Acc(0);
  for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
    for (int e = threadIdx.x; e < BM * BK; e += 256) {
      const int kk = e % BK, mm = e / BK;
      const int64_t m = m0 + mm, k = k0 + kk;
      As[kk][mm] = (m < p.M && k < p.K) ? static_cast<Acc>(load_as_math(A[m * p.a_sm + k * p.a_sk])) : Acc(0);
    }
    for (int e = threadIdx.x; e < BN * BK; e += 256) {
      const int nn = e % BN, kk = e / BN;
      const int64_t n = n0 + nn, k = k0 + kk;
      Bs[kk][nn] = (n < p.N && k < p.K) ? static_cast<Acc>(load_as_math(B[k * p.b_sk + n * p.b_sn])) : Acc(0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      Acc av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
    }
    __syncthreads();
  }
  const T* C = p.cin ? static_cast<const T*>(p.cin) + batch * p.c_sb : nullptr;
  T* O = static_cast<T*>(p.out) + batch * p.o_sb;
  const Acc alpha = static_cast<Acc>(p.alpha), beta = static_cast<Acc>(p.beta);
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < p.M && n < p.N) {
        Acc v = alpha * acc[i][j];
        if (C && p.beta != 0.0) v += beta * static_cast<Acc>(load_as_math(C[m * p.c_sm + n * p.c_sn]));
        O[m * p.o_sm + n * p.o_sn] = store_from_math<T>(static_cast<typename OpMath<T>::type>(v));
      }
    }
}

inline b200Status launch(const MatmulArgs& p, int32_t dtype, cudaStream_t s) {
  if (p.M == 0 || p.N == 0 || p.batch == 0) return B200_OK;
  const int64_t gx = (p.N + 63) / 64, gy = (p.M + 63) / 64;
  B200_REQUIRE(gy <= 65535 && p.batch <= 65535, B200_NOT_SUPPORTED, "matmul: shape too large for the SIMT path");
  dim3 grid(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(p.batch));
  switch (dtype) {
    case B200_F32: matmul_kernel<float, float><<<grid, 256, 0, s>>>(p); break;
    case B200_F64: matmul_kernel<double, double><<<grid, 256, 0, s>>>(p); break;
    case B200_BF16: matmul_kernel<bf16_t, float><<<grid, 256, 0, s>>>(p); break;
    case B200_F16: matmul_kernel<f16_t, float><<<grid, 256, 0, s>>>(p); break;
    default: return fail(B200_NOT_SUPPORTED, "matmul: dtype %d not supported", dtype);
  }
  return check_launch("matmul (simt)");
}

}  // namespace simt
}  // namespace b200
