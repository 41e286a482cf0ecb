// Latent attention of layer-list decoders (layerlist.cu): every token caches ONE row [c | k_r] - a normed latent c
// (kv_rank) and a rotated key part k_r (rot_dim) shared by all heads.  Head j's key is [Wuk_j c | k_r] and its
// value Wuv_j c, so with the query folded onto the latent, q~_j = [Wuk_j^T q_c | rot(q_r)], the score is
// q~_j . [c | k_r] and the output Wuv_j (sum_i p_i c_i): attention runs on the cache rows themselves, all heads
// of a token against the same rows, the value of a row being its first kv_rank entries.
//
//  * latent_prep_kernel        norms of the two latents, rotation of k_r, cache append (one CTA per token)
//  * latent_q_rope_kernel      rotated query part into the folded query
//  * head_gemm_kernel          batched per-head product (Wuk_j^T q_c and Wuv_j ctx): 64 x 64 FFMA tiles, 4 x 4 per thread;
//                              head_gemv_kernel for up to 8 rows (decode)
//  * attn_latent_kernel        flash-style exact attention: a CTA holds 32 (token, head) query rows in shared memory
//                              and walks the visible cache rows 32 at a time; a lane scores one key for its warp's
//                              four query rows, then the lanes own output columns.  Scores, weights and sums fp32.
//                              Decode splits the keys over CTAs; attn_latent_combine_kernel merges the parts.
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  for (int w = 0; w < nw; ++w) t += red[w];
  return t;
}

// pair (u, v) of entries (2i, 2i + 1) at position pos: (u cos a - v sin a, v cos a + u sin a), a = pos * f_i in fp32
__device__ __forceinline__ void rotate_pair(float u, float v, int pos, float f, float& ru, float& rv) {
  const float ang = (float)pos * f;
  float sn, cs;
  sincosf(ang, &sn, &cs);
  ru = u * cs - v * sn;
  rv = v * cs + u * sn;
}

template <typename KVT>
__global__ void __launch_bounds__(256) latent_prep_kernel(LatentPrepArgs a) {
  __shared__ float red[32];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const int b = r / a.L, t = r - b * a.L;
  const int pos = *a.pos_ptr + t;
  const float* row = a.proj + (size_t)r * a.ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) { const float v = row[i]; ss = fmaf(v, v, ss); }
  const float rq = 1.0f / sqrtf(block_sum(ss, red) / (float)a.q_rank + a.eps);
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) {
    const float v = row[i] * rq * a.wq[i];
    a.cq[(size_t)r * a.q_rank + i] = v;
    if (a.cq16) a.cq16[(size_t)r * a.q_rank + i] = __float2bfloat16_rn(v);
  }
  const float* kv = row + a.k_off;
  ss = 0.f;
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) { const float v = kv[i]; ss = fmaf(v, v, ss); }
  const float rk = 1.0f / sqrtf(block_sum(ss, red) / (float)a.kv_rank + a.eps);
  KVT* dst = (KVT*)a.cache + ((size_t)b * a.M + pos) * (a.kv_rank + a.rot_dim);
  for (int i = threadIdx.x; i < a.kv_rank; i += blockDim.x) dst[i] = from_f32<KVT>(kv[i] * rk * a.wk[i]);
  const float* kr = kv + a.kv_rank;
  for (int i = threadIdx.x; i < a.rot_dims / 2; i += blockDim.x) {
    float ru, rv;
    rotate_pair(kr[2 * i], kr[2 * i + 1], pos, a.inv_freq[i], ru, rv);
    dst[a.kv_rank + 2 * i] = from_f32<KVT>(ru);
    dst[a.kv_rank + 2 * i + 1] = from_f32<KVT>(rv);
  }
  for (int i = a.rot_dims + threadIdx.x; i < a.rot_dim; i += blockDim.x) dst[a.kv_rank + i] = from_f32<KVT>(kr[i]);
}

__global__ void latent_q_rope_kernel(const float* __restrict__ q, float* __restrict__ qlat, const float* __restrict__ inv_freq,
                                     const int* __restrict__ pos_ptr, int rows, int L, int H, int dim, int rot_dim, int rot_dims,
                                     int kv_rank) {
  pdl_launch();
  pdl_wait();
  const int half = (rot_dim + 1) / 2;  // work items per (row, head): one per pair, the tail entries one each
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * H * half) return;
  const int i = (int)(idx % half);
  const int64_t rh = idx / half;
  const int r = (int)(rh / H);
  const int pos = *pos_ptr + r % L;
  const float* src = q + rh * (dim + rot_dim) + dim;
  float* dst = qlat + rh * (kv_rank + rot_dim) + kv_rank;
  if (2 * i + 1 < rot_dims) {
    float ru, rv;
    rotate_pair(src[2 * i], src[2 * i + 1], pos, inv_freq[i], ru, rv);
    dst[2 * i] = ru;
    dst[2 * i + 1] = rv;
  } else {
    dst[2 * i] = src[2 * i];
    if (2 * i + 1 < rot_dim) dst[2 * i + 1] = src[2 * i + 1];
  }
}

// ---------------------------------------------------------------- batched per-head product
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16;

template <typename WT>
__global__ void __launch_bounds__(256) head_gemm_kernel(HeadGemmArgs a) {
  __shared__ __align__(16) float As[HG_BK][HG_BM + 4];
  __shared__ __align__(16) float Bs[HG_BK][HG_BN + 4];
  pdl_launch();
  pdl_wait();
  const int h = blockIdx.z, r0 = blockIdx.x * HG_BM, j0 = blockIdx.y * HG_BN;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  const float* A = a.A + (size_t)h * a.a_hs;
  const WT* W = (const WT*)a.W + (size_t)h * a.w_hs;
  float acc[4][4] = {};
  // a thread moves 4 elements of each tile; the next tile's global loads are issued ahead of this tile's products
  float ra[4], rb[4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = tid + u * 256;
      const int k = e & (HG_BK - 1), rr = e >> 4;
      const int r = r0 + rr, kk = k0 + k;
      ra[u] = (r < a.rows && kk < a.K) ? A[(size_t)r * a.lda + kk] : 0.f;
      int kb, jj;
      if (a.w_js == 1) { jj = e & (HG_BN - 1); kb = e >> 6; } else { kb = e & (HG_BK - 1); jj = e >> 4; }
      const int j = j0 + jj, kw = k0 + kb;
      rb[u] = (j < a.J && kw < a.K) ? to_f32(W[(size_t)kw * a.w_ks + (size_t)j * a.w_js]) : 0.f;
    }
  };
  fetch(0);
  for (int k0 = 0; k0 < a.K; k0 += HG_BK) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int e = tid + u * 256;
      As[e & (HG_BK - 1)][e >> 4] = ra[u];
      if (a.w_js == 1) Bs[e >> 6][e & (HG_BN - 1)] = rb[u]; else Bs[e & (HG_BK - 1)][e >> 4] = rb[u];
    }
    __syncthreads();
    if (k0 + HG_BK < a.K) fetch(k0 + HG_BK);
#pragma unroll
    for (int k = 0; k < HG_BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w}, br[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + ty * 4 + i;
    if (r >= a.rows) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int jj = j0 + tx * 4 + j;
      if (jj >= a.J) continue;
      const size_t o = (size_t)r * a.ldc + (size_t)h * a.c_hs + jj;
      a.C[o] = acc[i][j];
      if (a.C16) a.C16[o] = __float2bfloat16_rn(acc[i][j]);
    }
  }
}

// ---------------------------------------------------------------- attention over the latent cache
constexpr int LA_ROWS = 32, LA_KT = 32, LA_RW = 4, LA_WARPS = 8, LA_PF = 10;

__host__ __device__ inline int la_kstride(int Dk) {
  // 16-byte loads by 8 lanes at a time want an odd stride in 16-byte units; scalar loads an odd stride in words
  if (Dk % 4 == 0) return ((Dk / 4) & 1) ? Dk : Dk + 4;
  return (Dk & 1) ? Dk : Dk + 1;
}

// ND: output columns per lane (Dv <= 32 * ND)
template <typename KVT, int ND>
__global__ void __launch_bounds__(256) attn_latent_kernel(LatentAttnArgs a) {
  extern __shared__ __align__(16) float sm[];
  const int Dk = a.Dk, Dv = a.Dv, KS = la_kstride(Dk), QS = (Dk + 3) & ~3;
  float* Qs = sm;                                    // [LA_ROWS][QS]
  float* Ks = Qs + LA_ROWS * QS;                     // [LA_KT][KS]
  float* Ps = Ks + LA_KT * KS;                       // [LA_WARPS][LA_KT][LA_RW]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = blockIdx.y, split = blockIdx.z;
  const int nrow = a.L * a.H;                        // query rows of this sequence, (t, h) flattened
  const int row0 = blockIdx.x * LA_ROWS;
  const int pos0 = *a.pos_ptr;
  const int rows_here = min(LA_ROWS, nrow - row0);
  const int t_last = (row0 + rows_here - 1) / a.H;   // last token this CTA serves
  int k_begin = 0, k_end = pos0 + t_last + 1;        // visible keys of that token
  if (a.nsplit > 1) {
    const int per = ((k_end + a.nsplit - 1) / a.nsplit + LA_KT - 1) / LA_KT * LA_KT;
    k_begin = split * per;
    k_end = min(k_end, k_begin + per);
  }
  const float* qg = a.q + ((size_t)b * nrow + row0) * Dk;
  if (Dk % 4 == 0) {
    const int nv = LA_ROWS * Dk / 4;
#pragma unroll 4
    for (int v = threadIdx.x; v < nv; v += 256) {
      const int rr = (v * 4) / Dk, d = v * 4 - rr * Dk;
      float4 q4 = make_float4(0.f, 0.f, 0.f, 0.f);
      if (rr < rows_here) q4 = *reinterpret_cast<const float4*>(qg + (size_t)v * 4);
      *reinterpret_cast<float4*>(Qs + rr * QS + d) = make_float4(q4.x * a.scale, q4.y * a.scale, q4.z * a.scale, q4.w * a.scale);
    }
  } else {
#pragma unroll 8
    for (int e = threadIdx.x; e < LA_ROWS * Dk; e += 256) {
      const int rr = e / Dk, d = e - rr * Dk;
      Qs[rr * QS + d] = rr < rows_here ? qg[e] * a.scale : 0.f;
    }
  }
  // this warp's rows and their last visible key
  int lim[LA_RW];
#pragma unroll
  for (int i = 0; i < LA_RW; ++i) {
    const int rr = warp * LA_RW + i;
    lim[i] = rr < rows_here ? pos0 + (row0 + rr) / a.H : -1;
  }
  float mrun[LA_RW], lrun[LA_RW], acc[LA_RW][ND];
#pragma unroll
  for (int i = 0; i < LA_RW; ++i) {
    mrun[i] = -INFINITY; lrun[i] = 0.f;
#pragma unroll
    for (int c = 0; c < ND; ++c) acc[i][c] = 0.f;
  }
  const KVT* cb = (const KVT*)a.cache + (size_t)b * a.M * Dk;
  const bool vec4 = (Dk % 4) == 0;
  float* Pw = Ps + warp * LA_KT * LA_RW;
  // A tile of cache rows is one contiguous block.  With rows that are a whole number of 16-byte vectors every thread
  // keeps up to LA_PF vectors of the NEXT tile in registers: their loads are in flight while this tile is used.
  constexpr int VEC = 16 / (int)sizeof(KVT);
  const bool kvec = (Dk % VEC) == 0 && vec4;
  uint4 pf[LA_PF];
  auto issue = [&](int k0n) {
    const int nvec = min(LA_KT, k_end - k0n) * Dk / VEC;
    const KVT* srcn = cb + (size_t)k0n * Dk;
#pragma unroll
    for (int u = 0; u < LA_PF; ++u) {
      const int v = threadIdx.x + u * 256;
      if (v < nvec) pf[u] = ldg_stream16(srcn + (size_t)v * VEC);
    }
  };
  auto put = [&](const uint4& r, int v) {  // vector v of the tile: VEC entries of one row
    const int e = v * VEC, j = e / Dk, d = e - j * Dk;
    float f[VEC];
    Vec16<KVT>::unpack(r, f);
#pragma unroll
    for (int x = 0; x < VEC; x += 4) *reinterpret_cast<float4*>(Ks + j * KS + d + x) = make_float4(f[x], f[x + 1], f[x + 2], f[x + 3]);
  };
  if (kvec && k_begin < k_end) issue(k_begin);
  for (int k0 = k_begin; k0 < k_end; k0 += LA_KT) {
    const int nk = min(LA_KT, k_end - k0);
    __syncthreads();  // the previous tile is consumed (first pass: Qs is complete)
    const KVT* src = cb + (size_t)k0 * Dk;
    if (kvec) {
      const int nvec = nk * Dk / VEC;
#pragma unroll
      for (int u = 0; u < LA_PF; ++u) {
        const int v = threadIdx.x + u * 256;
        if (v < nvec) put(pf[u], v);
      }
      for (int v0 = threadIdx.x + LA_PF * 256; v0 < nvec; v0 += 4 * 256) {  // rows too long for the registers
        uint4 r[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) if (v0 + u * 256 < nvec) r[u] = ldg_stream16(src + (size_t)(v0 + u * 256) * VEC);
#pragma unroll
        for (int u = 0; u < 4; ++u) if (v0 + u * 256 < nvec) put(r[u], v0 + u * 256);
      }
    } else {
#pragma unroll 8
      for (int e = threadIdx.x; e < nk * Dk; e += 256) {
        const int j = e / Dk, d = e - j * Dk;
        Ks[j * KS + d] = to_f32(src[e]);
      }
    }
    __syncthreads();
    if (kvec && k0 + LA_KT < k_end) issue(k0 + LA_KT);
    // scores: lane = key
    float s[LA_RW] = {0.f, 0.f, 0.f, 0.f};
    if (lane < nk) {
      const float* kr = Ks + lane * KS;
      const float* q0 = Qs + (warp * LA_RW) * QS;
      if (vec4) {
        for (int d = 0; d < Dk; d += 4) {
          const float4 kv = *reinterpret_cast<const float4*>(kr + d);
#pragma unroll
          for (int i = 0; i < LA_RW; ++i) {
            const float4 qv = *reinterpret_cast<const float4*>(q0 + i * QS + d);
            s[i] = fmaf(qv.x, kv.x, s[i]); s[i] = fmaf(qv.y, kv.y, s[i]);
            s[i] = fmaf(qv.z, kv.z, s[i]); s[i] = fmaf(qv.w, kv.w, s[i]);
          }
        }
      } else {
        for (int d = 0; d < Dk; ++d) {
          const float kv = kr[d];
#pragma unroll
          for (int i = 0; i < LA_RW; ++i) s[i] = fmaf(q0[i * QS + d], kv, s[i]);
        }
      }
    }
    float p[LA_RW];
#pragma unroll
    for (int i = 0; i < LA_RW; ++i) {
      const bool vis = lane < nk && k0 + lane <= lim[i];
      const float sc = vis ? s[i] : -INFINITY;
      const float mnew = fmaxf(mrun[i], warp_max(sc));
      // a row that sees nothing yet keeps m = -inf: weights 0, no rescale
      p[i] = vis ? expf(sc - mnew) : 0.f;
      const float alpha = mnew == -INFINITY ? 1.f : expf(mrun[i] - mnew);
      lrun[i] = lrun[i] * alpha + warp_sum(p[i]);
      mrun[i] = mnew;
#pragma unroll
      for (int c = 0; c < ND; ++c) acc[i][c] *= alpha;
    }
    *reinterpret_cast<float4*>(Pw + lane * LA_RW) = make_float4(p[0], p[1], p[2], p[3]);
    __syncwarp();
    for (int j = 0; j < nk; ++j) {
      const float4 pj = *reinterpret_cast<const float4*>(Pw + j * LA_RW);
      const float* vr = Ks + j * KS;
#pragma unroll
      for (int c = 0; c < ND; ++c) {
        const int d = lane + 32 * c;
        const float v = d < Dv ? vr[d] : 0.f;
        acc[0][c] = fmaf(pj.x, v, acc[0][c]); acc[1][c] = fmaf(pj.y, v, acc[1][c]);
        acc[2][c] = fmaf(pj.z, v, acc[2][c]); acc[3][c] = fmaf(pj.w, v, acc[3][c]);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int i = 0; i < LA_RW; ++i) {
    const int rr = warp * LA_RW + i;
    if (rr >= rows_here) continue;
    const size_t row = (size_t)b * nrow + row0 + rr;           // = token row * H + head
    if (a.nsplit > 1) {
      float* po = a.part_o + (row * a.nsplit + split) * Dv;
#pragma unroll
      for (int c = 0; c < ND; ++c) { const int d = lane + 32 * c; if (d < Dv) po[d] = acc[i][c]; }
      if (lane == 0) { a.part_ml[(row * a.nsplit + split) * 2] = mrun[i]; a.part_ml[(row * a.nsplit + split) * 2 + 1] = lrun[i]; }
    } else {
      const size_t tok = row / a.H;
      const int head = (int)(row - tok * a.H);
      const float g = a.gate ? 1.0f / (1.0f + expf(-a.gate[tok * a.ld_gate + head])) : 1.0f;
      const float inv = g / lrun[i];
#pragma unroll
      for (int c = 0; c < ND; ++c) { const int d = lane + 32 * c; if (d < Dv) a.out[row * Dv + d] = acc[i][c] * inv; }
    }
  }
}

__global__ void __launch_bounds__(128) attn_latent_combine_kernel(LatentAttnArgs a) {
  __shared__ float wsplit[64];
  pdl_launch();
  pdl_wait();
  const size_t row = blockIdx.x;
  const float* ml = a.part_ml + row * a.nsplit * 2;
  float mx = -INFINITY;
  for (int s = 0; s < a.nsplit; ++s) mx = fmaxf(mx, ml[2 * s]);
  if (threadIdx.x < a.nsplit) wsplit[threadIdx.x] = ml[2 * threadIdx.x] == -INFINITY ? 0.f : expf(ml[2 * threadIdx.x] - mx);
  __syncthreads();
  float l = 0.f;
  for (int s = 0; s < a.nsplit; ++s) l = fmaf(wsplit[s], ml[2 * s + 1], l);
  const size_t tok = row / a.H;
  const int head = (int)(row - tok * a.H);
  const float g = a.gate ? 1.0f / (1.0f + expf(-a.gate[tok * a.ld_gate + head])) : 1.0f;
  const float inv = g / l;
  const float* po = a.part_o + row * a.nsplit * a.Dv;
  for (int d = threadIdx.x; d < a.Dv; d += blockDim.x) {
    float o = 0.f;
#pragma unroll 8
    for (int s = 0; s < a.nsplit; ++s) o = fmaf(wsplit[s], po[(size_t)s * a.Dv + d], o);
    a.out[row * a.Dv + d] = o * inv;
  }
}

// Few rows (decode): the per-head product as matrix-vector products that stream the head's weights once.
// w_ks == 1 (an output's weights are contiguous): a warp per output; w_js == 1: a thread per output, the k loop unrolled.
template <typename WT>
__global__ void __launch_bounds__(256) head_gemv_kernel(HeadGemmArgs a) {
  pdl_launch();
  pdl_wait();
  const int h = blockIdx.y, r = blockIdx.z, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* A = a.A + (size_t)r * a.lda + (size_t)h * a.a_hs;
  const WT* W = (const WT*)a.W + (size_t)h * a.w_hs;
  float v;
  int j;
  if (a.w_ks == 1) {
    j = blockIdx.x * 8 + warp;
    if (j >= a.J) return;
    const WT* wr = W + (size_t)j * a.w_js;
    float acc = 0.f;
#pragma unroll 4
    for (int k = lane; k < a.K; k += 32) acc = fmaf(to_f32(wr[k]), A[k], acc);
    v = warp_sum(acc);
    if (lane != 0) return;
  } else {
    j = blockIdx.x * 256 + threadIdx.x;
    if (j >= a.J) return;
    float acc = 0.f;
#pragma unroll 8
    for (int k = 0; k < a.K; ++k) acc = fmaf(to_f32(W[(size_t)k * a.w_ks + j]), A[k], acc);
    v = acc;
  }
  const size_t o = (size_t)r * a.ldc + (size_t)h * a.c_hs + j;
  a.C[o] = v;
  if (a.C16) a.C16[o] = __float2bfloat16_rn(v);
}

template <typename KVT>
cudaError_t launch_la(const LatentAttnArgs& a, cudaStream_t s) {
  const int nrow = a.L * a.H;
  const dim3 grid((nrow + LA_ROWS - 1) / LA_ROWS, a.B, std::max(1, a.nsplit));
  const size_t smem = latent_attn_smem(a.Dk);
  const int nd = (a.Dv + 31) / 32;
#define LA_CASE(N)                                                                                                        \
  if (nd <= N) {                                                                                                          \
    static bool set = false;                                                                                              \
    if (!set) {                                                                                                           \
      cudaFuncSetAttribute(attn_latent_kernel<KVT, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);          \
      set = true;                                                                                                         \
    }                                                                                                                     \
    return launch_k(attn_latent_kernel<KVT, N>, grid, dim3(256), smem, s, a);                                             \
  }
  LA_CASE(1) LA_CASE(2) LA_CASE(4) LA_CASE(8) LA_CASE(16) LA_CASE(32)
#undef LA_CASE
  return cudaErrorInvalidValue;
}

}  // namespace

size_t latent_attn_smem(int Dk) {
  return ((size_t)LA_ROWS * ((Dk + 3) & ~3) + (size_t)LA_KT * la_kstride(Dk) + LA_WARPS * LA_KT * LA_RW) * sizeof(float);
}

bool latent_attn_supported(int Dk, int Dv) { return Dv >= 1 && Dv <= Dk && Dv <= 1024 && latent_attn_smem(Dk) <= 220 * 1024; }

cudaError_t launch_latent_attn(const LatentAttnArgs& a, bool kv_bf16, cudaStream_t s) {
  cudaError_t e = kv_bf16 ? launch_la<bf16>(a, s) : launch_la<float>(a, s);
  if (e != cudaSuccess || a.nsplit <= 1) return e;
  return launch_k(attn_latent_combine_kernel, dim3(a.B * a.L * a.H), dim3(128), 0, s, a);
}

cudaError_t launch_latent_prep(const LatentPrepArgs& a, int rows, bool kv_bf16, cudaStream_t s) {
  if (kv_bf16) return launch_k(latent_prep_kernel<bf16>, dim3(rows), dim3(256), 0, s, a);
  return launch_k(latent_prep_kernel<float>, dim3(rows), dim3(256), 0, s, a);
}

cudaError_t launch_latent_q_rope(const float* q, float* qlat, const float* inv_freq, const int* pos_ptr, int rows, int L,
                                 int H, int dim, int rot_dim, int rot_dims, int kv_rank, cudaStream_t s) {
  const int64_t n = (int64_t)rows * H * ((rot_dim + 1) / 2);
  return launch_k(latent_q_rope_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, q, qlat, inv_freq, pos_ptr, rows, L, H,
                  dim, rot_dim, rot_dims, kv_rank);
}

cudaError_t launch_head_gemm(const HeadGemmArgs& a, bool w_bf16, cudaStream_t s) {
  if (a.rows <= 8) {
    const dim3 g(a.w_ks == 1 ? (a.J + 7) / 8 : (a.J + 255) / 256, a.H, a.rows);
    if (w_bf16) return launch_k(head_gemv_kernel<bf16>, g, dim3(256), 0, s, a);
    return launch_k(head_gemv_kernel<float>, g, dim3(256), 0, s, a);
  }
  const dim3 grid((a.rows + HG_BM - 1) / HG_BM, (a.J + HG_BN - 1) / HG_BN, a.H);
  if (w_bf16) return launch_k(head_gemm_kernel<bf16>, grid, dim3(256), 0, s, a);
  return launch_k(head_gemm_kernel<float>, grid, dim3(256), 0, s, a);
}
