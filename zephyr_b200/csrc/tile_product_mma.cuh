// One CTA's tile of a product  Y[r, n] = sum_k A[r, k] * W[n, k]  on the tensor cores (mma.sync m16n8k16,
// bfloat16 operands, float32 sums), for products whose rows are picked row by row: tokens gathered for
// an expert, one head's columns of a wider row.  The weights are bfloat16; the rows of A are bfloat16 or
// float32 (rounded to bfloat16 as they are staged).
//
// 256 threads = 8 warps on a tile of TM_BM = 64 rows by TM_BN = 64 outputs, walked in steps of TM_BK = 32
// along k: warp w owns rows 16 (w & 3) .. + 16 and outputs 32 (w >> 2) .. + 32, four m16n8 tiles.  With
// DUAL two weight matrices share the staged rows of A (a gate and an up projection).  Rows of shared
// memory are padded by 8 elements, which spreads the fragment loads over all banks.
#pragma once

#include "mma.cuh"

namespace zb {

constexpr int TM_BM = 64;
constexpr int TM_BN = 64;
constexpr int TM_BK = 32;
constexpr int TM_LD = TM_BK + 8;
constexpr int TM_THREADS = 256;

struct TileMmaSmem {
  __align__(16) __nv_bfloat16 a[TM_BM][TM_LD];
  __align__(16) __nv_bfloat16 b[2][TM_BN][TM_LD];
  const void* row[TM_BM];     // where each row of A begins (null: a row past the end, read as zeros)
};

__device__ __forceinline__ uint4 tm_load8(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
__device__ __forceinline__ uint4 tm_load8(const float* p) {
  const float4 lo = *reinterpret_cast<const float4*>(p), hi = *reinterpret_cast<const float4*>(p + 4);
  return make_uint4(pack_bf16(lo.x, lo.y), pack_bf16(lo.z, lo.w), pack_bf16(hi.x, hi.y), pack_bf16(hi.z, hi.w));
}

// Eight elements of a row at column k (zeros where the row is absent or the columns lie beyond K).
// `vectors`: every row starts on a 16-byte (bfloat16) or 32-byte (float32) boundary and K is a multiple of 8.
template <typename TA>
__device__ __forceinline__ uint4 tm_row_piece(const TA* row, int k, int K, bool vectors) {
  if (row == nullptr || k >= K) return make_uint4(0, 0, 0, 0);
  if (vectors) return tm_load8(row + k);
  float v[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) v[u] = k + u < K ? to_float(row[k + u]) : 0.0f;
  return make_uint4(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]), pack_bf16(v[4], v[5]), pack_bf16(v[6], v[7]));
}

// acc[s][nt][c]: weight matrix s (the second only with DUAL), n8 tile nt of the warp's 32 outputs, c as in
// the m16n8 accumulator: row g (+ 8 for c >= 2), column 2 t + (c & 1), with g = lane / 4, t = lane % 4.
template <bool DUAL, typename TA>
__device__ __forceinline__ void tile_product_mma(TileMmaSmem& sm, const __nv_bfloat16* w0, const __nv_bfloat16* w1,
                                                 int n_left, int K, bool a_vectors, bool w_vectors,
                                                 float (&acc)[2][4][4], bool interleaved = false) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3, m0 = (warp & 3) * 16, n0 = (warp >> 2) * 32;
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[s][nt][c] = 0.0f;
  const int r = tid >> 2, piece = (tid & 3) * 8;         // this thread stages 8 columns of row r (A) and of output r (W)
  const TA* a_row = static_cast<const TA*>(sm.row[r]);
  const bool real = r < n_left;
  // `interleaved`: the matrices' rows alternate in blocks of 8 (row r of each lies 16 (r / 8) + r % 8 rows in).
  const size_t w_row = interleaved ? static_cast<size_t>((r >> 3) * 16 + (r & 7)) : static_cast<size_t>(r);
  const __nv_bfloat16* w0_row = real ? w0 + w_row * K : nullptr;
  const __nv_bfloat16* w1_row = DUAL && real ? w1 + w_row * K : nullptr;
  // The pieces of the step after this one are asked for before this step's products, so that their
  // way from memory runs beside the tensor cores' work.
  uint4 av = tm_row_piece(a_row, piece, K, a_vectors);
  uint4 bv0 = tm_row_piece(w0_row, piece, K, w_vectors);
  uint4 bv1 = make_uint4(0, 0, 0, 0);
  if (DUAL) bv1 = tm_row_piece(w1_row, piece, K, w_vectors);
  for (int k0 = 0; k0 < K; k0 += TM_BK) {
    __syncthreads();                                      // the step before is no longer read
    *reinterpret_cast<uint4*>(&sm.a[r][piece]) = av;
    *reinterpret_cast<uint4*>(&sm.b[0][r][piece]) = bv0;
    if (DUAL) *reinterpret_cast<uint4*>(&sm.b[1][r][piece]) = bv1;
    __syncthreads();
    if (k0 + TM_BK < K) {
      av = tm_row_piece(a_row, k0 + TM_BK + piece, K, a_vectors);
      bv0 = tm_row_piece(w0_row, k0 + TM_BK + piece, K, w_vectors);
      if (DUAL) bv1 = tm_row_piece(w1_row, k0 + TM_BK + piece, K, w_vectors);
    }
#pragma unroll
    for (int kk = 0; kk < TM_BK; kk += 16) {
      unsigned a[4];
      a[0] = *reinterpret_cast<const unsigned*>(&sm.a[m0 + g][kk + 2 * t]);
      a[1] = *reinterpret_cast<const unsigned*>(&sm.a[m0 + g + 8][kk + 2 * t]);
      a[2] = *reinterpret_cast<const unsigned*>(&sm.a[m0 + g][kk + 2 * t + 8]);
      a[3] = *reinterpret_cast<const unsigned*>(&sm.a[m0 + g + 8][kk + 2 * t + 8]);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const int n = n0 + nt * 8 + g;
        mma_bf16_16816(acc[0][nt], a, *reinterpret_cast<const unsigned*>(&sm.b[0][n][kk + 2 * t]),
                       *reinterpret_cast<const unsigned*>(&sm.b[0][n][kk + 2 * t + 8]));
        if (DUAL)
          mma_bf16_16816(acc[1][nt], a, *reinterpret_cast<const unsigned*>(&sm.b[1][n][kk + 2 * t]),
                         *reinterpret_cast<const unsigned*>(&sm.b[1][n][kk + 2 * t + 8]));
      }
    }
  }
}

// Row and column, inside the tile, of accumulator element (nt, c) of this thread.
__device__ __forceinline__ int tm_row(int c) { return ((threadIdx.x >> 5) & 3) * 16 + ((threadIdx.x & 31) >> 2) + (c >= 2 ? 8 : 0); }
__device__ __forceinline__ int tm_col(int nt, int c) {
  return (threadIdx.x >> 7) * 32 + nt * 8 + 2 * (threadIdx.x & 3) + (c & 1);
}

inline bool tm_aligned(const void* p, size_t bytes) { return reinterpret_cast<uintptr_t>(p) % bytes == 0; }

}  // namespace zb
