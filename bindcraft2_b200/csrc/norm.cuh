// LayerNorm kernels (memory-bound): one warp per row, 128-bit loads, warp-shuffle reductions, two-pass variance in
// fp32 (reference arithmetic: bindcraft/af/alphafold/model/common_modules.py:127-184, eps 1e-5).
//
//   ln_fwd_kernel      x fp32 [M,C] -> y bf16 [M,C]; optionally also the attention pair bias  nb[h][pos] = y . wb[:,h]
//   ln_bwd_kernel      dx = LN'(x)^T (dy + sum_h dnb[h][pos] wb[:,h]);  g_out = g_in + dx  (fp32 cotangent stream)
//   cln_fwd_kernel     centre norm of the triangle multiplication: channel-major bf16 planes [C][M] -> row-major y [M,C]
//   cln_bwd_kernel     its backward: (t planes, dy rows) -> dt planes
#pragma once
#include "common.cuh"

namespace bc2 {

template <int C>
struct RowVec {
  static constexpr int VPL = C / 32;             // values per lane
  static constexpr int VEC = VPL >= 4 ? 4 : VPL;  // values per vector access
  static constexpr int NV = VPL / VEC;
  // element index of value (i, j) held by `lane`
  __device__ static __forceinline__ int idx(int lane, int i, int j) { return i * (32 * VEC) + lane * VEC + j; }
};

template <int C>
__device__ __forceinline__ void load_row_f32(const float* p, int lane, float (&v)[C / 32]) {
  using R = RowVec<C>;
#pragma unroll
  for (int i = 0; i < R::NV; ++i) {
    if constexpr (R::VEC == 4) {
      float4 t = *reinterpret_cast<const float4*>(p + R::idx(lane, i, 0));
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    } else if constexpr (R::VEC == 2) {
      float2 t = *reinterpret_cast<const float2*>(p + R::idx(lane, i, 0));
      v[2 * i] = t.x; v[2 * i + 1] = t.y;
    } else {
      v[i] = p[R::idx(lane, i, 0)];
    }
  }
}
template <int C>
__device__ __forceinline__ void store_row_f32(float* p, int lane, const float (&v)[C / 32]) {
  using R = RowVec<C>;
#pragma unroll
  for (int i = 0; i < R::NV; ++i) {
    if constexpr (R::VEC == 4)
      *reinterpret_cast<float4*>(p + R::idx(lane, i, 0)) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    else if constexpr (R::VEC == 2)
      *reinterpret_cast<float2*>(p + R::idx(lane, i, 0)) = make_float2(v[2 * i], v[2 * i + 1]);
    else
      p[R::idx(lane, i, 0)] = v[i];
  }
}
template <int C>
__device__ __forceinline__ void load_row_bf16(const bf16* p, int lane, float (&v)[C / 32]) {
  using R = RowVec<C>;
#pragma unroll
  for (int i = 0; i < R::NV; ++i) {
    if constexpr (R::VEC == 4) {
      uint2 t = *reinterpret_cast<const uint2*>(p + R::idx(lane, i, 0));
      float2 a = unpack_bf16(t.x), b = unpack_bf16(t.y);
      v[4 * i] = a.x; v[4 * i + 1] = a.y; v[4 * i + 2] = b.x; v[4 * i + 3] = b.y;
    } else if constexpr (R::VEC == 2) {
      float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(p + R::idx(lane, i, 0)));
      v[2 * i] = a.x; v[2 * i + 1] = a.y;
    } else {
      v[i] = __bfloat162float(p[R::idx(lane, i, 0)]);
    }
  }
}
template <int C>
__device__ __forceinline__ void store_row_bf16(bf16* p, int lane, const float (&v)[C / 32]) {
  using R = RowVec<C>;
#pragma unroll
  for (int i = 0; i < R::NV; ++i) {
    if constexpr (R::VEC == 4)
      *reinterpret_cast<uint2*>(p + R::idx(lane, i, 0)) = make_uint2(pack_bf16(v[4 * i], v[4 * i + 1]), pack_bf16(v[4 * i + 2], v[4 * i + 3]));
    else if constexpr (R::VEC == 2)
      *reinterpret_cast<uint32_t*>(p + R::idx(lane, i, 0)) = pack_bf16(v[2 * i], v[2 * i + 1]);
    else
      p[R::idx(lane, i, 0)] = __float2bfloat16(v[i]);
  }
}

template <int C>
__device__ __forceinline__ void row_stats(const float (&v)[C / 32], float& mean, float& rstd) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < C / 32; ++i) s += v[i];
  mean = warp_sum(s) * (1.f / C);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < C / 32; ++i) {
    float d = v[i] - mean;
    q += d * d;
  }
  rstd = rsqrtf(warp_sum(q) * (1.f / C) + 1e-5f);
}

// Index of the attention-bias entry that row m = (i, j) of an [n,n] pair tensor produces.  The attention kernels keep
// the bias as [head][KEY][query] (a warp's 32 query rows then read consecutive floats).  Row-wise attention uses
// bias(q = i, k = j), stored at j*n + i; the ending-node attention is built from the transposed activations
// (modules.py:696-720), bias(q = j, k = i), stored at i*n + j = m.
__device__ __forceinline__ long bias_pos(int m, int n, int transposed) {
  if (transposed) return m;
  const int i = m / n, j = m - i * n;
  return (long)j * n + i;
}

struct LnArgs {
  const float* x = nullptr;     // [M, C] fp32
  const float* scale = nullptr; // [C]
  const float* offset = nullptr;
  bf16* y = nullptr;            // [M, ldy] or null
  long ldy = 0;
  const float* wb = nullptr;    // [H, C] bias projection (head-major) or null
  float* nb = nullptr;          // [H][M]
  int H = 0, n = 0, transposed = 0;
  int relu = 0;  // y = max(LN(x), 0)
  int M = 0;
};

constexpr int LN_MAXH = 8;

// Persistent: each warp keeps scale, offset and its slice of the bias projection in registers and strides over rows.
template <int C>
__global__ void __launch_bounds__(256) ln_fwd_kernel(LnArgs a) {
  using R = RowVec<C>;
  const int lane = threadIdx.x & 31;
  const int nwarp = gridDim.x * 8;
  float sc[R::VPL], of[R::VPL];
  load_row_f32<C>(a.scale, lane, sc);
  load_row_f32<C>(a.offset, lane, of);
  float wbr[LN_MAXH][R::VPL];
  if (a.wb) {
#pragma unroll
    for (int h = 0; h < LN_MAXH; ++h)
      if (h < a.H) load_row_f32<C>(a.wb + (long)h * C, lane, wbr[h]);
  }
  int m = blockIdx.x * 8 + (threadIdx.x >> 5);
  float vn[R::VPL];  // next row, loaded one iteration ahead so two rows are in flight per warp
  if (m < a.M) load_row_f32<C>(a.x + (long)m * C, lane, vn);
  for (; m < a.M; m += nwarp) {
    float v[R::VPL];
#pragma unroll
    for (int i = 0; i < R::VPL; ++i) v[i] = vn[i];
    if (m + nwarp < a.M) load_row_f32<C>(a.x + (long)(m + nwarp) * C, lane, vn);
    float mean, rstd;
    row_stats<C>(v, mean, rstd);
#pragma unroll
    for (int i = 0; i < R::VPL; ++i) v[i] = (v[i] - mean) * rstd * sc[i] + of[i];
    if (a.relu) {
#pragma unroll
      for (int i = 0; i < R::VPL; ++i) v[i] = fmaxf(v[i], 0.f);
    }
    if (a.y) store_row_bf16<C>(a.y + (long)m * a.ldy, lane, v);
    if (a.wb) {
      const long pos = bias_pos(m, a.n, a.transposed);
      float mine = 0.f;  // lane h ends up holding head h's dot product
#pragma unroll
      for (int h = 0; h < LN_MAXH; ++h)
        if (h < a.H) {
          float s = 0.f;
#pragma unroll
          for (int i = 0; i < R::VPL; ++i) s += v[i] * wbr[h][i];
          s = warp_sum(s);
          if (lane == h) mine = s;
        }
      if (lane < a.H) a.nb[(long)lane * a.M + pos] = mine;
    }
  }
}

struct LnBwdArgs {
  const float* x = nullptr;      // [M, C] forward input of the norm
  const float* scale = nullptr;
  const bf16* dy = nullptr;      // [M, ldy] gradient wrt the norm output, or null
  long ldy = 0;
  const float* wb = nullptr;     // [H, C]
  const float* dnb = nullptr;    // [H][M] gradient wrt the bias
  int H = 0, n = 0, transposed = 0;
  const float* g_in = nullptr;   // [M, C] running cotangent or null
  float* g_out = nullptr;        // [M, C]
  int M = 0;
};

template <int C>
__global__ void __launch_bounds__(256) ln_bwd_kernel(LnBwdArgs a) {
  using R = RowVec<C>;
  const int lane = threadIdx.x & 31;
  const int nwarp = gridDim.x * 8;
  float sc[R::VPL];
  load_row_f32<C>(a.scale, lane, sc);
  float wbr[LN_MAXH][R::VPL];
  if (a.wb) {
#pragma unroll
    for (int h = 0; h < LN_MAXH; ++h)
      if (h < a.H) load_row_f32<C>(a.wb + (long)h * C, lane, wbr[h]);
  }
  int m = blockIdx.x * 8 + (threadIdx.x >> 5);
  float vn[R::VPL], dn[R::VPL], gn[R::VPL];  // next row's operands, loaded one iteration ahead
  auto load_next = [&](int mm) {
    load_row_f32<C>(a.x + (long)mm * C, lane, vn);
    if (a.dy) load_row_bf16<C>(a.dy + (long)mm * a.ldy, lane, dn);
    if (a.g_in) load_row_f32<C>(a.g_in + (long)mm * C, lane, gn);
  };
#pragma unroll
  for (int i = 0; i < R::VPL; ++i) dn[i] = gn[i] = 0.f;
  if (m < a.M) load_next(m);
  for (; m < a.M; m += nwarp) {
    float v[R::VPL], d[R::VPL], g[R::VPL];
#pragma unroll
    for (int i = 0; i < R::VPL; ++i) {
      v[i] = vn[i];
      d[i] = dn[i];
      g[i] = gn[i];
    }
    if (m + nwarp < a.M) load_next(m + nwarp);
    if (a.wb) {
      const long pos = bias_pos(m, a.n, a.transposed);
      const float mine = lane < a.H ? a.dnb[(long)lane * a.M + pos] : 0.f;
#pragma unroll
      for (int h = 0; h < LN_MAXH; ++h)
        if (h < a.H) {
          const float gb = __shfl_sync(0xffffffffu, mine, h);
#pragma unroll
          for (int i = 0; i < R::VPL; ++i) d[i] += gb * wbr[h][i];
        }
    }
    float mean, rstd;
    row_stats<C>(v, mean, rstd);
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < R::VPL; ++i) {
      v[i] = (v[i] - mean) * rstd;  // xhat
      d[i] *= sc[i];                // dxhat
      s1 += d[i];
      s2 += d[i] * v[i];
    }
    s1 = warp_sum(s1) * (1.f / C);
    s2 = warp_sum(s2) * (1.f / C);
#pragma unroll
    for (int i = 0; i < R::VPL; ++i) g[i] += rstd * (d[i] - s1 - v[i] * s2);
    store_row_f32<C>(a.g_out + (long)m * C, lane, g);
  }
}

template <int C>
inline void ln_fwd(const LnArgs& a, cudaStream_t st) {
  launch_counter()++; ln_fwd_kernel<C><<<std::min(cdiv(a.M, 8), 148 * 8), 256, 0, st>>>(a);
}
template <int C>
inline void ln_bwd(const LnBwdArgs& a, cudaStream_t st) {
  launch_counter()++; ln_bwd_kernel<C><<<std::min(cdiv(a.M, 8), 148 * 8), 256, 0, st>>>(a);
}

// ------------------------------------------------------------------------------------------- centre norm (transposing)
// t: [C][M] bf16 planes.  A block stages a [C x 64-position] tile through shared memory (reads coalesced along
// positions), then each warp normalises whole positions and writes row-major (coalesced along channels).
template <int C>
__global__ void __launch_bounds__(256) cln_fwd_kernel(const bf16* __restrict__ t, const float* __restrict__ scale,
                                                      const float* __restrict__ offset, bf16* __restrict__ y, int M) {
  __shared__ float tile[C][65];
  const int p0 = blockIdx.x * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = warp; c < C; c += 8) {
    const int p = p0 + 2 * lane;
    float2 f = make_float2(0.f, 0.f);
    if (p < M) f = unpack_bf16(*reinterpret_cast<const uint32_t*>(t + (long)c * M + p));
    tile[c][2 * lane] = f.x;
    tile[c][2 * lane + 1] = f.y;
  }
  __syncthreads();
  constexpr int VPL = C / 32;
  for (int r = warp; r < 64; r += 8) {
    const int p = p0 + r;
    if (p >= M) break;
    float v[VPL];
#pragma unroll
    for (int i = 0; i < VPL; ++i) v[i] = tile[i * 32 + lane][r];
    float mean, rstd;
    row_stats<C>(v, mean, rstd);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int c = i * 32 + lane;
      y[(long)p * C + c] = __float2bfloat16((v[i] - mean) * rstd * scale[c] + offset[c]);
    }
  }
}

// dt[c][p] = rstd * (dy*scale - mean(dy*scale) - that * mean(dy*scale*that))
template <int C>
__global__ void __launch_bounds__(256) cln_bwd_kernel(const bf16* __restrict__ t, const float* __restrict__ scale,
                                                      const bf16* __restrict__ dy, bf16* __restrict__ dt, int M) {
  __shared__ float tile[C][65];
  const int p0 = blockIdx.x * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = warp; c < C; c += 8) {
    const int p = p0 + 2 * lane;
    float2 f = make_float2(0.f, 0.f);
    if (p < M) f = unpack_bf16(*reinterpret_cast<const uint32_t*>(t + (long)c * M + p));
    tile[c][2 * lane] = f.x;
    tile[c][2 * lane + 1] = f.y;
  }
  __syncthreads();
  constexpr int VPL = C / 32;
  for (int r = warp; r < 64; r += 8) {
    const int p = p0 + r;
    if (p < M) {
      float v[VPL], d[VPL];
#pragma unroll
      for (int i = 0; i < VPL; ++i) v[i] = tile[i * 32 + lane][r];
      float mean, rstd;
      row_stats<C>(v, mean, rstd);
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < VPL; ++i) {
        const int c = i * 32 + lane;
        v[i] = (v[i] - mean) * rstd;
        d[i] = __bfloat162float(dy[(long)p * C + c]) * scale[c];
        s1 += d[i];
        s2 += d[i] * v[i];
      }
      s1 = warp_sum(s1) * (1.f / C);
      s2 = warp_sum(s2) * (1.f / C);
#pragma unroll
      for (int i = 0; i < VPL; ++i) tile[i * 32 + lane][r] = rstd * (d[i] - s1 - v[i] * s2);
    }
  }
  __syncthreads();
  for (int c = warp; c < C; c += 8) {
    const int p = p0 + 2 * lane;
    if (p < M) *reinterpret_cast<uint32_t*>(dt + (long)c * M + p) = pack_bf16(tile[c][2 * lane], tile[c][2 * lane + 1]);
  }
}

}  // namespace bc2
