// One CTA's tile of a product  Y[r, n] = sum_k A[r, k] * W[n, k]  on CUDA cores, float32 sums in the
// order of k, for products whose rows are picked row by row (tokens gathered for an expert, one head's
// columns of a wider row).  Both element types take this path; it is the true 32-bit product of such
// layers and the general one for bfloat16 shapes the tensor-core tile (tile_product_mma.cuh) refuses.
//
// 256 threads; a tile is TP_BM rows by TP_BN outputs, walked in steps of TP_BK along k.  Thread
// (ty, tx) = (tid / 16, tid % 16) owns rows 2 ty, 2 ty + 1 and outputs tx + 16 j, j < 4.
#pragma once

#include "common.cuh"

namespace zb {

constexpr int TP_BM = 32;
constexpr int TP_BN = 64;
constexpr int TP_BK = 32;
constexpr int TP_THREADS = 256;

struct TileProductSmem {
  float a[TP_BM][TP_BK + 1];
  float b[2][TP_BN][TP_BK + 1];
  const void* row[TP_BM];     // where each row of A begins (null: a row past the end, read as zeros)
};

// acc[m][s][j]: row 2 ty + m, weight matrix s (the second only with DUAL), output tx + 16 j.
// `w0` / `w1` point at the first output row of the tile ([n, K] with rows K apart); `n_left` outputs
// and K columns are real, the rest reads as zeros.
// The rows of A are of type TA (they may be float32 beside bfloat16 weights), the weights of type T.
template <typename T, bool DUAL, typename TA = T>
__device__ __forceinline__ void tile_product(TileProductSmem& sm, const T* w0, const T* w1, int n_left, int K,
                                             float (&acc)[2][2][4], bool interleaved = false) {
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int s = 0; s < 2; ++s)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[m][s][j] = 0.0f;
  for (int k0 = 0; k0 < K; k0 += TP_BK) {
    __syncthreads();
    for (int e = tid; e < TP_BM * TP_BK; e += TP_THREADS) {
      const int r = e / TP_BK, c = e - r * TP_BK;
      const TA* src = static_cast<const TA*>(sm.row[r]);
      sm.a[r][c] = (src != nullptr && k0 + c < K) ? to_float(src[k0 + c]) : 0.0f;
    }
    for (int e = tid; e < TP_BN * TP_BK; e += TP_THREADS) {
      const int n = e / TP_BK, c = e - n * TP_BK;
      const bool ok = n < n_left && k0 + c < K;
      // `interleaved`: the matrices' rows alternate in blocks of 8 (row n of each lies 16 (n / 8) + n % 8 rows in).
      const size_t row = interleaved ? static_cast<size_t>((n >> 3) * 16 + (n & 7)) : static_cast<size_t>(n);
      sm.b[0][n][c] = ok ? to_float(w0[row * K + k0 + c]) : 0.0f;
      if (DUAL) sm.b[1][n][c] = ok ? to_float(w1[row * K + k0 + c]) : 0.0f;
    }
    __syncthreads();
#pragma unroll 8
    for (int c = 0; c < TP_BK; ++c) {
      const float a0 = sm.a[2 * ty][c], a1 = sm.a[2 * ty + 1][c];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float b = sm.b[0][tx + 16 * j][c];
        acc[0][0][j] = fmaf(a0, b, acc[0][0][j]);
        acc[1][0][j] = fmaf(a1, b, acc[1][0][j]);
        if (DUAL) {
          const float b2 = sm.b[1][tx + 16 * j][c];
          acc[0][1][j] = fmaf(a0, b2, acc[0][1][j]);
          acc[1][1][j] = fmaf(a1, b2, acc[1][1][j]);
        }
      }
    }
  }
}

}  // namespace zb
