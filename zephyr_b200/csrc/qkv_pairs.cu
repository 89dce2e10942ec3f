// From a fused q/k/v projection to queries and cache entries, for attention whose rotation turns
// adjacent pairs: bias, per-head RMS norm of q and k, rotation, and the write of k and v into the
// pages, in one pass and in float32 with a single rounding at the store.
//
//   x = projection + bias                                  (q, k and v)
//   x = x / sqrt(mean(x^2) + eps) * w                      (q and k; w shared by the heads)
//   (x[2i], x[2i+1]) <- (x[2i] c - x[2i+1] s, x[2i+1] c + x[2i] s),  c, s = cos, sin(p * f[i])
//                                                          (q and k; i < rot_dims / 2, the rest passes)
//
// with p the token's position and f a table of float32 frequencies the host made.  Keys and values
// may differ in width: a page holds [nkv][page_size][kd] keys and behind them [nkv][page_size][vd]
// values; rows whose bytes are a multiple of 16 are stored with permuted 16-byte chunks (common.cuh:
// kv_swizzle), any other width as it is.  One warp per (token, head); a lane owns adjacent pairs.
//
// Further forms, each a parameter: a norm without scales (`unit_norm`: x / sqrt(mean(x^2) + eps) on q and
// k); values that are the keys as projected, before their norm (`values_from_keys`: the projection has
// no value columns); a multiplier on the normed queries that grows with the position,
// 1 + coef * ln(floor((p + 1) / every) + 1) (`q_temp_*`); a cache that keeps keys only (vd = 0: its
// reader takes the keys for values too); and no query heads at all (nh = 0: only the cache is written).
#include "common.cuh"

namespace zb {

constexpr int QP_WARPS = 4;
constexpr int QP_MAX_PAIRS = 8;    // pairs per lane: widths up to 512; a launch takes 1, 2, 4 or 8 by its widest head

struct QkvPairsArgs {
  void* q_out;               // [T, nh * kd]
  const void* qkv;           // [T, stride]: q heads, k heads, v heads
  long long stride;
  const float* bias;         // null or [nh*kd + nkv*kd + nkv*vd]
  const float* q_norm_w;     // null or [kd]
  const float* k_norm_w;     // null or [kd]
  float eps;
  const float* freqs;        // null or [rot_dims / 2]
  int rot_dims;
  const int* positions;
  const int* token_row;
  void* cache;               // null: only the queries are made
  const int* block_table;
  int max_blocks, page_size, num_pages, num_rows;
  int nh, nkv, kd, vd;
  int unit_norm;             // q and k are normed without scales (q_norm_w and k_norm_w are null)
  int values_from_keys;      // the value head j is the key head j's columns, un-normed
  float q_temp_coef;         // 0: no multiplier on the queries
  int q_temp_every;
  int pairs_aligned;         // every pair of the projection, the bias and the scales may move as one 8-byte value
  int* status;
};

__device__ __forceinline__ void load_pair(const float* p, bool aligned, float& a, float& b) {
  if (aligned) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x; b = v.y;
  } else {
    a = p[0]; b = p[1];
  }
}
__device__ __forceinline__ void load_pair(const __nv_bfloat16* p, bool aligned, float& a, float& b) {
  a = __bfloat162float(p[0]); b = __bfloat162float(p[1]);
}
__device__ __forceinline__ void store_pair(float* p, float a, float b) { *reinterpret_cast<float2*>(p) = make_float2(a, b); }
__device__ __forceinline__ void store_pair(__nv_bfloat16* p, float a, float b) {
  *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(a, b);
}

template <typename IN, typename T, int QP_PAIRS>
__global__ void __launch_bounds__(QP_WARPS * 32) qkv_pairs_kernel(const QkvPairsArgs a) {
  const int t = blockIdx.x, lane = threadIdx.x & 31;
  const int head = blockIdx.y * QP_WARPS + (threadIdx.x >> 5);
  const int total = a.cache != nullptr ? a.nh + (a.vd > 0 ? 2 : 1) * a.nkv : a.nh;
  if (head >= total) return;
  const bool is_q = head < a.nh, is_k = !is_q && head < a.nh + a.nkv;
  const int dim = (is_q || is_k) ? a.kd : a.vd;
  const long long col = is_q ? static_cast<long long>(head) * a.kd
                      : is_k ? static_cast<long long>(a.nh) * a.kd + static_cast<long long>(head - a.nh) * a.kd
                      : a.values_from_keys
                          ? static_cast<long long>(a.nh) * a.kd + static_cast<long long>(head - a.nh - a.nkv) * a.kd
                          : static_cast<long long>(a.nh + a.nkv) * a.kd +
                                static_cast<long long>(head - a.nh - a.nkv) * a.vd;
  const IN* src = static_cast<const IN*>(a.qkv) + static_cast<long long>(t) * a.stride + col;
  const int pos = a.positions[t];

  float x[QP_PAIRS][2];
  float ss = 0.0f;
#pragma unroll
  for (int k = 0; k < QP_PAIRS; ++k) {
    const int i = 2 * (lane + 32 * k);
    x[k][0] = x[k][1] = 0.0f;
    if (i + 1 < dim) {
      load_pair(src + i, a.pairs_aligned != 0, x[k][0], x[k][1]);
      if (a.bias != nullptr) {
        float b0, b1;
        load_pair(a.bias + col + i, a.pairs_aligned != 0, b0, b1);
        x[k][0] += b0; x[k][1] += b1;
      }
      ss += x[k][0] * x[k][0] + x[k][1] * x[k][1];
    } else if (i < dim) {
      x[k][0] = to_float(src[i]) + (a.bias != nullptr ? a.bias[col + i] : 0.0f);
      ss += x[k][0] * x[k][0];
    }
  }
  {
    const float* w = is_q ? a.q_norm_w : (is_k ? a.k_norm_w : nullptr);
    if (w == nullptr && a.unit_norm && (is_q || is_k)) {
      const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(dim) + a.eps);
#pragma unroll
      for (int k = 0; k < QP_PAIRS; ++k) {
        x[k][0] *= inv;
        x[k][1] *= inv;
      }
    }
    if (w != nullptr) {
      const float inv = 1.0f / sqrtf(warp_sum(ss) / static_cast<float>(dim) + a.eps);
#pragma unroll
      for (int k = 0; k < QP_PAIRS; ++k) {
        const int i = 2 * (lane + 32 * k);
        if (i + 1 < dim) {
          float w0, w1;
          load_pair(w + i, a.pairs_aligned != 0, w0, w1);
          x[k][0] = x[k][0] * inv * w0;
          x[k][1] = x[k][1] * inv * w1;
        } else if (i < dim) {
          x[k][0] = x[k][0] * inv * w[i];
        }
      }
    }
  }
  if ((is_q || is_k) && a.freqs != nullptr) {
#pragma unroll
    for (int k = 0; k < QP_PAIRS; ++k) {
      const int i = 2 * (lane + 32 * k);
      if (i + 1 < a.rot_dims) {
        float s, c;
        sincosf(static_cast<float>(pos) * a.freqs[i >> 1], &s, &c);
        const float u = x[k][0], v = x[k][1];
        x[k][0] = u * c - v * s;
        x[k][1] = v * c + u * s;
      }
    }
  }

  if (is_q && a.q_temp_coef != 0.0f) {
    const float m = 1.0f + a.q_temp_coef * logf(static_cast<float>((pos + 1) / a.q_temp_every) + 1.0f);
#pragma unroll
    for (int k = 0; k < QP_PAIRS; ++k) {
      x[k][0] *= m;
      x[k][1] *= m;
    }
  }

  T* dst;
  int swizzle_pos = -1;          // -1: the row is stored as it is
  if (is_q) {
    dst = static_cast<T*>(a.q_out) + (static_cast<long long>(t) * a.nh + head) * a.kd;
  } else {
    const int row = a.token_row[t], block = pos / a.page_size;
    if (row < 0 || row >= a.num_rows || block >= a.max_blocks) {
      if (lane == 0) report(a.status, STATUS_ROW_OUT_OF_RANGE, row, t);
      return;
    }
    const int page = a.block_table[static_cast<long long>(row) * a.max_blocks + block];
    if (page <= 0 || page >= a.num_pages) {      // page 0 is the null page and is never written
      if (lane == 0) report(a.status, STATUS_PAGE_OUT_OF_RANGE, page, t);
      return;
    }
    const int kvh = is_k ? head - a.nh : head - a.nh - a.nkv;
    const long long page_elems = static_cast<long long>(a.nkv) * a.page_size * (a.kd + a.vd);
    const long long part = is_k ? 0 : static_cast<long long>(a.nkv) * a.page_size * a.kd;
    dst = static_cast<T*>(a.cache) + static_cast<long long>(page) * page_elems + part +
          (static_cast<long long>(kvh) * a.page_size + pos % a.page_size) * dim;
    if ((dim * static_cast<int>(sizeof(T))) % 16 == 0) swizzle_pos = pos;
  }
#pragma unroll
  for (int k = 0; k < QP_PAIRS; ++k) {
    const int i = 2 * (lane + 32 * k);
    if (i < dim) {
      const int at = swizzle_pos >= 0 ? kv_element_index(i, swizzle_pos, dim, sizeof(T)) : i;
      if (i + 1 < dim && a.pairs_aligned) {
        store_pair(dst + at, x[k][0], x[k][1]);                    // a pair never straddles a 16-byte chunk
      } else {
        dst[at] = from_float<T>(x[k][0]);
        if (i + 1 < dim) dst[at + 1] = from_float<T>(x[k][1]);
      }
    }
  }
}

}  // namespace zb

using namespace zb;

ZB_API int zb_qkv_pairs(void* q_out, const void* qkv, long long stride, const float* bias, const float* q_norm_w,
                        const float* k_norm_w, float eps, const float* freqs, int rot_dims, const int* positions,
                        const int* token_row, void* cache, const int* block_table, int max_blocks, int page_size,
                        int num_pages, int num_rows, int tokens, int nh, int nkv, int kd, int vd, int unit_norm,
                        int values_from_keys, float q_temp_coef, int q_temp_every, int in_dtype, int dtype,
                        int* status, void* stream) {
  if (tokens < 0 || nh < 0 || nkv <= 0 || kd <= 0 || vd < 0 || rot_dims < 0 || rot_dims > kd || rot_dims % 2 != 0 ||
      page_size <= 0 || (nh == 0 && cache == nullptr) || (values_from_keys && vd != kd) ||
      (q_temp_coef != 0.0f && q_temp_every <= 0) ||
      (unit_norm && (q_norm_w != nullptr || k_norm_w != nullptr)))
    return ERR_BAD_ARGUMENT;
  if (kd > 64 * QP_MAX_PAIRS || vd > 64 * QP_MAX_PAIRS) return ERR_UNSUPPORTED;
  if (tokens == 0) return OK;
  QkvPairsArgs a;
  a.q_out = q_out; a.qkv = qkv; a.stride = stride; a.bias = bias; a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w;
  a.eps = eps; a.freqs = freqs; a.rot_dims = freqs != nullptr ? rot_dims : 0; a.positions = positions;
  a.token_row = token_row; a.cache = cache; a.block_table = block_table; a.max_blocks = max_blocks;
  a.page_size = page_size; a.num_pages = num_pages; a.num_rows = num_rows; a.nh = nh; a.nkv = nkv; a.kd = kd;
  a.vd = vd; a.status = status;
  a.unit_norm = unit_norm; a.values_from_keys = values_from_keys; a.q_temp_coef = q_temp_coef;
  a.q_temp_every = q_temp_every;
  auto even = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 8 == 0; };
  a.pairs_aligned = kd % 2 == 0 && vd % 2 == 0 && stride % 2 == 0 && even(qkv) && even(bias) && even(q_norm_w) &&
                    even(k_norm_w) && even(q_out) && even(cache);
  const int heads = cache != nullptr ? nh + (vd > 0 ? 2 : 1) * nkv : nh;
  const dim3 grid(tokens, (heads + QP_WARPS - 1) / QP_WARPS);
  auto s = static_cast<cudaStream_t>(stream);
  if (dtype == DTYPE_F32 && in_dtype != DTYPE_F32) return ERR_BAD_ARGUMENT;
  const int widest = kd > vd ? kd : vd;
#define ZB_QP(PAIRS)                                                                                         \
  {                                                                                                          \
    if (dtype == DTYPE_F32) qkv_pairs_kernel<float, float, PAIRS><<<grid, QP_WARPS * 32, 0, s>>>(a);          \
    else if (in_dtype == DTYPE_F32) qkv_pairs_kernel<float, __nv_bfloat16, PAIRS><<<grid, QP_WARPS * 32, 0, s>>>(a); \
    else qkv_pairs_kernel<__nv_bfloat16, __nv_bfloat16, PAIRS><<<grid, QP_WARPS * 32, 0, s>>>(a);             \
  }
  if (widest <= 64) ZB_QP(1)
  else if (widest <= 128) ZB_QP(2)
  else if (widest <= 256) ZB_QP(4)
  else ZB_QP(8)
#undef ZB_QP
  return launch_result();
}
