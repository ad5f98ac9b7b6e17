// Matrix product on the CUDA cores with 32-bit accumulation:
//   out[M, N] = x[rows[m] or m, :K] . w[N, K]^T (+ bias[N])
// (turingserve/ops/reference.py:45-47 `F.linear`; the output head of turingserve/model/qwen2.py:94-99
// when `rows` selects the sampled rows and the output type is float).
//
// This is the float32 path's product (true 32-bit: FFMA only, no tensor-core mode) and the
// fallback for shapes the tensor-core kernels refuse.  Each output element is accumulated over k
// in ascending order whatever M is, so a row's result does not depend on its batch-mates.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(TO* __restrict__ out, const TI* __restrict__ x, const TI* __restrict__ w,
                 const TI* __restrict__ bias, const int* __restrict__ rows, int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;       // loader: row 0..63, k offset 0,4,8,12
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};

  const int am = m0 + lr;
  const TI* a_row = nullptr;
  if (am < M) a_row = x + (size_t)(rows != nullptr ? rows[am] : am) * K;
  const int wn = n0 + lr;
  const TI* w_row = wn < N ? w + (size_t)wn * K : nullptr;

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_row != nullptr && k < K) ? to_f(a_row[k]) : 0.f;
      Ws[lk + i][lr] = (w_row != nullptr && k < K) ? to_f(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (bias != nullptr) v += to_f(bias[n]);
      out[(size_t)m * N + n] = from_f<TO>(v);
    }
  }
}

}  // namespace

TS_API int ts_linear_simt(void* out, const void* x, const void* w, const void* bias, const int* rows,
                          int M, int N, int K, int dtype, int out_dtype, void* stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_linear: K = %d", K);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(ceil_div(N, BN), ceil_div(M, BM));
  if (grid.y > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_linear: M = %d too large for one launch", M);
  if (dtype == TS_F32 && out_dtype == TS_F32)
    ts_launch(gemm_simt_kernel<float, float>, dim3(grid), dim3(256), 0, s, (float*)out, (const float*)x, (const float*)w,
                                                        (const float*)bias, rows, M, N, K);
  else if (dtype == TS_BF16 && out_dtype == TS_BF16)
    ts_launch(gemm_simt_kernel<bf16, bf16>, dim3(grid), dim3(256), 0, s, (bf16*)out, (const bf16*)x, (const bf16*)w,
                                                      (const bf16*)bias, rows, M, N, K);
  else if (dtype == TS_BF16 && out_dtype == TS_F32)
    ts_launch(gemm_simt_kernel<bf16, float>, dim3(grid), dim3(256), 0, s, (float*)out, (const bf16*)x, (const bf16*)w,
                                                       (const bf16*)bias, rows, M, N, K);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_linear: dtype %d -> %d", dtype, out_dtype);
  TS_LAUNCH_CHECK();
}
