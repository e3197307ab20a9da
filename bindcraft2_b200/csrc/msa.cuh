// MSA-track kernels that are not plain GEMMs: the outer product mean (reassociated, reference
// bindcraft/af/alphafold/model/modules.py:1128-1213) and the per-column attention over alignment depth S <= 8
// (modules.py:566-616), each forward and backward.  The alignment is shallow in design runs (S = 1..8), so these are
// bandwidth/latency-bound CUDA-core kernels with coalesced accesses along the channel axis.
#pragma once
#include "common.cuh"

namespace bc2 {

constexpr int OPM_C = 32;   // num_outer_channel
constexpr int OPM_F = 128;  // pair channels (c_z)

// lr: [S*N][64] bf16 = masked left (cols 0..31) | masked right (cols 32..63) projections.
// tmp[s][j][c][f] = sum_e right[s,j,e] * W[c,e,f]          (W: output_w [32,32,128] fp32)
__global__ void __launch_bounds__(128) opm_tmp_kernel(const bf16* __restrict__ lr, const float* __restrict__ W,
                                                      float* __restrict__ tmp, int SN) {
  __shared__ float r[OPM_C];
  const int sj = blockIdx.x, c = blockIdx.y, f = threadIdx.x;
  if (threadIdx.x < OPM_C) r[threadIdx.x] = __bfloat162float(lr[(long)sj * 64 + 32 + threadIdx.x]);
  __syncthreads();
  float acc = 0.f;
#pragma unroll
  for (int e = 0; e < OPM_C; ++e) acc += r[e] * W[((long)c * OPM_C + e) * OPM_F + f];
  tmp[((long)sj * OPM_C + c) * OPM_F + f] = acc;
}

// pair_out[i,j,f] = pair_in[i,j,f] + (sum_{s,c} left[s,i,c] tmp[s,j,c,f] + b[f]) / (1e-3 + sum_s m[s,i] m[s,j])
// block = (j, 32-row i tile), thread = f.
__global__ void __launch_bounds__(128)
opm_out_kernel(const bf16* __restrict__ lr, const float* __restrict__ tmp, const float* __restrict__ bias,
               const float* __restrict__ msa_mask, const float* __restrict__ pair_in, float* __restrict__ pair_out, int S,
               int N) {
  extern __shared__ __align__(16) float sl[];  // [32][S*32] left tile, then [32] norms
  const int j = blockIdx.x, i0 = blockIdx.y * 32, f = threadIdx.x;
  const int K = S * OPM_C;
  float* snorm = sl + 32 * K;
  for (int t = threadIdx.x; t < 32 * K; t += 128) {
    const int ii = t / K, k = t % K, s = k / OPM_C, c = k % OPM_C;
    sl[t] = (i0 + ii < N) ? __bfloat162float(lr[((long)s * N + i0 + ii) * 64 + c]) : 0.f;
  }
  if (threadIdx.x < 32) {
    float nrm = 0.f;
    if (i0 + threadIdx.x < N)
      for (int s = 0; s < S; ++s) nrm += msa_mask[(long)s * N + i0 + threadIdx.x] * msa_mask[(long)s * N + j];
    snorm[threadIdx.x] = 1.f / (1e-3f + nrm);
  }
  __syncthreads();
  float acc[32];
#pragma unroll
  for (int ii = 0; ii < 32; ++ii) acc[ii] = 0.f;
  // four k per step: one 128-bit shared-memory broadcast feeds four FMAs (K = 32 S is a multiple of 4)
  const float4* sl4 = reinterpret_cast<const float4*>(sl);
  for (int k = 0; k < K; k += 4) {
    const int s = k / OPM_C, c = k % OPM_C;
    const float* tp = tmp + (((long)s * N + j) * OPM_C + c) * OPM_F + f;
    const float t0 = tp[0], t1 = tp[OPM_F], t2 = tp[2 * OPM_F], t3 = tp[3 * OPM_F];
#pragma unroll
    for (int ii = 0; ii < 32; ++ii) {
      const float4 l = sl4[(ii * K + k) >> 2];
      acc[ii] += l.x * t0 + l.y * t1 + l.z * t2 + l.w * t3;
    }
  }
  const float b = bias[f];
#pragma unroll
  for (int ii = 0; ii < 32; ++ii) {
    const int i = i0 + ii;
    if (i < N) {
      const long idx = ((long)i * N + j) * OPM_F + f;
      pair_out[idx] = pair_in[idx] + (acc[ii] + b) * snorm[ii];
    }
  }
}

// Backward.  d_out[i,j,f] = g[i,j,f] / (1e-3 + norm[i,j]).
// d_left[s,i,c] = sum_{j,f} d_out[i,j,f] tmp[s,j,c,f]      block = (tile of OPM_IT rows i, s, slice of j); 8 warps stride
// over j, lanes over f.  Each tmp value read feeds OPM_IT rows, which divides the L2 traffic on tmp by OPM_IT.
constexpr int OPM_IT = 4;
__global__ void __launch_bounds__(256)
opm_dleft_kernel(const float* __restrict__ g, const float* __restrict__ tmp, const float* __restrict__ msa_mask,
                 float* __restrict__ dlr /*[S*N][64] fp32, zeroed by the caller*/, int S, int N) {
  __shared__ float red[8][OPM_IT][OPM_C];
  const int i0 = blockIdx.x * OPM_IT, s = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float acc[OPM_IT][OPM_C];
#pragma unroll
  for (int r = 0; r < OPM_IT; ++r)
#pragma unroll
    for (int c = 0; c < OPM_C; ++c) acc[r][c] = 0.f;
  for (int j = warp + 8 * blockIdx.z; j < N; j += 8 * gridDim.z) {
    float4 d[OPM_IT];
#pragma unroll
    for (int r = 0; r < OPM_IT; ++r) {
      const int i = min(i0 + r, N - 1);
      float nrm = 0.f;
      for (int ss = 0; ss < S; ++ss) nrm += msa_mask[(long)ss * N + i] * msa_mask[(long)ss * N + j];
      const float inv = (i0 + r < N) ? 1.f / (1e-3f + nrm) : 0.f;
      d[r] = *reinterpret_cast<const float4*>(g + ((long)i * N + j) * OPM_F + lane * 4);
      d[r].x *= inv; d[r].y *= inv; d[r].z *= inv; d[r].w *= inv;
    }
    const float* tp = tmp + ((long)s * N + j) * OPM_C * OPM_F + lane * 4;
#pragma unroll
    for (int c = 0; c < OPM_C; ++c) {
      const float4 t = *reinterpret_cast<const float4*>(tp + c * OPM_F);
#pragma unroll
      for (int r = 0; r < OPM_IT; ++r) acc[r][c] += d[r].x * t.x + d[r].y * t.y + d[r].z * t.z + d[r].w * t.w;
    }
  }
#pragma unroll
  for (int r = 0; r < OPM_IT; ++r)
#pragma unroll
    for (int c = 0; c < OPM_C; ++c) {
      const float v = warp_sum(acc[r][c]);
      if (lane == 0) red[warp][r][c] = v;
    }
  __syncthreads();
  if (threadIdx.x < OPM_IT * OPM_C) {
    const int r = threadIdx.x / OPM_C, c = threadIdx.x % OPM_C;
    if (i0 + r < N) {
      float v = 0.f;
      for (int w = 0; w < 8; ++w) v += red[w][r][c];
      atomicAdd(&dlr[((long)s * N + i0 + r) * 64 + c], v);  // gridDim.z blocks share a row; dlr starts at zero
    }
  }
}

// d_tmp[s,j,c,f] = sum_i left[s,i,c] d_out[i,j,f]          block = (j, s), thread = f, acc over c
__global__ void __launch_bounds__(128)
opm_dtmp_kernel(const float* __restrict__ g, const bf16* __restrict__ lr, const float* __restrict__ msa_mask,
                float* __restrict__ dtmp, int S, int N) {
  __shared__ __align__(16) float sl[32][OPM_C + 4];  // rows padded to a multiple of 16 bytes for 128-bit reads
  __shared__ float sinv[32];
  const int j = blockIdx.x, s = blockIdx.y, f = threadIdx.x;
  float acc[OPM_C];
#pragma unroll
  for (int c = 0; c < OPM_C; ++c) acc[c] = 0.f;
  for (int i0 = 32 * blockIdx.z; i0 < N; i0 += 32 * gridDim.z) {
    __syncthreads();
    for (int t = threadIdx.x; t < 32 * OPM_C; t += 128) {
      const int ii = t / OPM_C, c = t % OPM_C;
      sl[ii][c] = (i0 + ii < N) ? __bfloat162float(lr[((long)s * N + i0 + ii) * 64 + c]) : 0.f;
    }
    if (threadIdx.x < 32) {
      float nrm = 0.f;
      if (i0 + threadIdx.x < N)
        for (int ss = 0; ss < S; ++ss) nrm += msa_mask[(long)ss * N + i0 + threadIdx.x] * msa_mask[(long)ss * N + j];
      sinv[threadIdx.x] = 1.f / (1e-3f + nrm);
    }
    __syncthreads();
    for (int ii = 0; ii < 32 && i0 + ii < N; ++ii) {
      const float d = g[((long)(i0 + ii) * N + j) * OPM_F + f] * sinv[ii];
#pragma unroll
      for (int c = 0; c < OPM_C; c += 4) {
        const float4 l = *reinterpret_cast<const float4*>(&sl[ii][c]);
        acc[c] += l.x * d; acc[c + 1] += l.y * d; acc[c + 2] += l.z * d; acc[c + 3] += l.w * d;
      }
    }
  }
#pragma unroll
  for (int c = 0; c < OPM_C; ++c)  // gridDim.z blocks each hold a slice of the sum over i; dtmp starts at zero
    atomicAdd(&dtmp[(((long)s * N + j) * OPM_C + c) * OPM_F + f], acc[c]);
}

// d_right[s,j,e] = sum_{c,f} d_tmp[s,j,c,f] W[c,e,f]       block = (s,j), warp per e-group, lanes over f
__global__ void __launch_bounds__(256)
opm_dright_kernel(const float* __restrict__ dtmp, const float* __restrict__ W, float* __restrict__ dlr, int SN) {
  const int sj = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < OPM_C; e += 8) {
    float acc = 0.f;
    for (int c = 0; c < OPM_C; ++c) {
      const float4 d = *reinterpret_cast<const float4*>(dtmp + ((long)sj * OPM_C + c) * OPM_F + lane * 4);
      const float4 w = *reinterpret_cast<const float4*>(W + ((long)c * OPM_C + e) * OPM_F + lane * 4);
      acc += d.x * w.x + d.y * w.y + d.z * w.z + d.w * w.w;
    }
    acc = warp_sum(acc);
    if (lane == 0) dlr[(long)sj * 64 + 32 + e] = acc;
  }
}

// d(lr) fp32 -> bf16 with the row mask applied (lr = mask * (x W + b))
__global__ void opm_dlr_store_kernel(const float* __restrict__ dlr, const float* __restrict__ msa_mask,
                                     bf16* __restrict__ out, long n) {
  const long t = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) out[t] = __float2bfloat16(dlr[t] * msa_mask[t / 64]);
}

// ------------------------------------------------------------------------------------------- MSA column attention
// qkvg: [S*N][4*H*D] (q scaled | k | v | sigmoid gate), row = s*N + n.  One warp per (n, h); lanes over d (D = 32).
// Forward writes og = softmax(q k^T + 1e9(mask-1)) v * gate  [S*N][H*D].
template <int MAXS>
__global__ void __launch_bounds__(256)
msacol_fwd_kernel(const bf16* __restrict__ qkvg, const float* __restrict__ msa_mask, bf16* __restrict__ og, int S, int N,
                  int H) {
  const int lane = threadIdx.x & 31;
  const long w = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= (long)N * H) return;
  const int n = w / H, h = w % H;
  const int HD = H * 32;
  const long ld = 4 * HD;
  float k[MAXS], v[MAXS], mb[MAXS];
#pragma unroll
  for (int s = 0; s < MAXS; ++s)
    if (s < S) {
      const long row = (long)s * N + n;
      k[s] = __bfloat162float(qkvg[row * ld + HD + h * 32 + lane]);
      v[s] = __bfloat162float(qkvg[row * ld + 2 * HD + h * 32 + lane]);
      mb[s] = 1e9f * (msa_mask[row] - 1.f);
    }
#pragma unroll
  for (int sq = 0; sq < MAXS; ++sq)
    if (sq < S) {
      const long row = (long)sq * N + n;
      const float q = __bfloat162float(qkvg[row * ld + h * 32 + lane]);
      float lg[MAXS], mx = -INFINITY;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          lg[s] = fminf(fmaxf(warp_sum(q * k[s]) + mb[s], -1e8f), 1e8f);
          mx = fmaxf(mx, lg[s]);
        }
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          const float p = __expf(lg[s] - mx);
          l += p;
          o += p * v[s];
        }
      const float g = __bfloat162float(qkvg[row * ld + 3 * HD + h * 32 + lane]);
      og[row * HD + h * 32 + lane] = __float2bfloat16(o / l * g);
    }
}

// Backward: recomputes the S x S probabilities; d_og [S*N][H*D] -> d_qkvg [S*N][4*H*D] (dq | dk | dv | d gate-pre).
template <int MAXS>
__global__ void __launch_bounds__(256)
msacol_bwd_kernel(const bf16* __restrict__ qkvg, const float* __restrict__ msa_mask, const bf16* __restrict__ d_og,
                  bf16* __restrict__ d_qkvg, int S, int N, int H) {
  const int lane = threadIdx.x & 31;
  const long w = (long)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (w >= (long)N * H) return;
  const int n = w / H, h = w % H;
  const int HD = H * 32;
  const long ld = 4 * HD;
  float k[MAXS], v[MAXS], mb[MAXS], dk[MAXS], dv[MAXS];
#pragma unroll
  for (int s = 0; s < MAXS; ++s)
    if (s < S) {
      const long row = (long)s * N + n;
      k[s] = __bfloat162float(qkvg[row * ld + HD + h * 32 + lane]);
      v[s] = __bfloat162float(qkvg[row * ld + 2 * HD + h * 32 + lane]);
      mb[s] = 1e9f * (msa_mask[row] - 1.f);
      dk[s] = dv[s] = 0.f;
    }
#pragma unroll
  for (int sq = 0; sq < MAXS; ++sq)
    if (sq < S) {
      const long row = (long)sq * N + n;
      const float q = __bfloat162float(qkvg[row * ld + h * 32 + lane]);
      float lg[MAXS], p[MAXS], mx = -INFINITY;
      bool live[MAXS];
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          const float raw = warp_sum(q * k[s]) + mb[s];
          live[s] = raw >= -1e8f && raw <= 1e8f;
          lg[s] = fminf(fmaxf(raw, -1e8f), 1e8f);
          mx = fmaxf(mx, lg[s]);
        }
      float l = 0.f, o = 0.f;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          p[s] = __expf(lg[s] - mx);
          l += p[s];
          o += p[s] * v[s];
        }
      const float inv = 1.f / l;
      o *= inv;
      const float g = __bfloat162float(qkvg[row * ld + 3 * HD + h * 32 + lane]);
      const float dg = __bfloat162float(d_og[row * HD + h * 32 + lane]);
      const float d_o = dg * g;
      d_qkvg[row * ld + 3 * HD + h * 32 + lane] = __float2bfloat16(dg * o * g * (1.f - g));
      const float delta = warp_sum(d_o * o);
      float dq = 0.f;
#pragma unroll
      for (int s = 0; s < MAXS; ++s)
        if (s < S) {
          const float ps = p[s] * inv;
          const float dp = warp_sum(d_o * v[s]);
          const float ds = live[s] ? ps * (dp - delta) : 0.f;
          dq += ds * k[s];
          dk[s] += ds * q;
          dv[s] += ps * d_o;
        }
      d_qkvg[row * ld + h * 32 + lane] = __float2bfloat16(dq);
    }
#pragma unroll
  for (int s = 0; s < MAXS; ++s)
    if (s < S) {
      const long row = (long)s * N + n;
      d_qkvg[row * ld + HD + h * 32 + lane] = __float2bfloat16(dk[s]);
      d_qkvg[row * ld + 2 * HD + h * 32 + lane] = __float2bfloat16(dv[s]);
    }
}

}  // namespace bc2
