// Matrix-state recurrences over time for the recurrent token mixers of layer-list decoders: linear attention
// with a fixed decay per head, and the gated delta rule with a decay per head and key channel.  One fp32
// state matrix S [DK, DV] per (sequence slot, head), carried in HBM between calls.
//
//   mode 0   S <- decay_h S + k v^T                                   o = S^T q
//   mode 1   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T    o = S^T q   (o sees this token's write)
//
// The columns of S never mix: column j needs v_j, the token's k, q, g (shared by all columns) and nothing of
// any other column.  So a CTA owns a tile of CPB columns of one (slot, head) for the whole call; a column is
// held by TPC adjacent lanes, each with R rows of it in registers (row i = lane + r TPC), and the two inner
// products over the key dimension are R FMAs plus log2(TPC) shuffles.  Tokens are staged TCH at a time in
// shared memory by the whole CTA (coalesced), outputs leave the same way.  The state is read once at the
// start and written once at the end: a decode step (L = 1) moves 2 x DK x DV x 4 bytes per head and nothing
// else of size - it is HBM-bound on the state; a prompt is a dependent chain over its tokens, the same
// arithmetic in the same order however the prompt is cut into calls, so cutting it changes no bit.
#include <algorithm>

#include "common.cuh"
#include "mixer.h"

namespace {

template <int R, int MODE>
__global__ void __launch_bounds__(256) recur_kernel(RecurArgs a, int TPC, int CPB, int TCH) {
  extern __shared__ float sm[];
  const int DKP = R * TPC;  // padded key dimension: rows >= DK hold zeros
  float* sq = sm;                                   // [TCH][DKP]
  float* sk = sq + (size_t)TCH * DKP;               // [TCH][DKP]
  float* sg = sk + (size_t)TCH * DKP;               // [TCH][DKP]   (mode 1)
  float* sv = sg + (MODE == 1 ? (size_t)TCH * DKP : 0);  // [TCH][CPB]
  float* so = sv + (size_t)TCH * CPB;               // [TCH][CPB]
  float* sb = so + (size_t)TCH * CPB;               // [TCH]        (mode 1)
  pdl_launch();
  pdl_wait();
  const int tid = threadIdx.x, nthr = blockDim.x;
  const int ntile = (a.DV + CPB - 1) / CPB;
  const int h = blockIdx.x / ntile, tile = blockIdx.x - h * ntile, b = blockIdx.y;
  const int kvh = h / a.rep;
  const int cl = tid / TPC, s = tid - cl * TPC;
  const int j = tile * CPB + cl;
  const bool live = cl < CPB;  // a CTA is padded to a whole warp when CPB * TPC < 32
  const bool col_ok = live && j < a.DV;
  float* Sg = a.state + ((size_t)b * a.H + h) * a.DK * a.DV;
  float S[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = s + r * TPC;
    S[r] = (col_ok && i < a.DK) ? Sg[(size_t)i * a.DV + j] : 0.f;
  }
  const float lam = MODE == 0 ? a.head_decay[h] : 0.f;

  for (int t0 = 0; t0 < a.L; t0 += TCH) {
    const int n = min(TCH, a.L - t0);
    __syncthreads();  // the previous chunk's outputs have left
    for (int idx = tid; idx < n * DKP; idx += nthr) {
      const int tok = idx / DKP, i = idx - tok * DKP;
      const size_t row = (size_t)b * a.L + t0 + tok;
      float qv = 0.f, kv = 0.f, gv = 0.f;
      if (i < a.DK) {
        qv = a.q[row * a.ld_q + (size_t)kvh * a.DK + i];
        kv = a.k[row * a.ld_k + (size_t)kvh * a.DK + i];
        if (a.act_in) { qv = silu_ref(qv); kv = silu_ref(kv); }
        if (MODE == 1) gv = a.g[row * ((size_t)a.H * a.DK) + (size_t)h * a.DK + i];
      }
      sq[idx] = qv;
      sk[idx] = kv;
      if (MODE == 1) sg[idx] = gv;
    }
    for (int idx = tid; idx < n * CPB; idx += nthr) {
      const int tok = idx / CPB, c = idx - tok * CPB;
      const int jj = tile * CPB + c;
      float vv = 0.f;
      if (jj < a.DV) {
        vv = a.v[((size_t)b * a.L + t0 + tok) * a.ld_v + (size_t)h * a.DV + jj];
        if (a.act_in) vv = silu_ref(vv);
      }
      sv[idx] = vv;
    }
    if (MODE == 1)
      for (int tok = tid; tok < n; tok += nthr) sb[tok] = a.beta[((size_t)b * a.L + t0 + tok) * a.H + h];
    __syncthreads();

    for (int tok = 0; tok < n; ++tok) {
      const float* qk = sq + (size_t)tok * DKP + s;
      const float* kk = sk + (size_t)tok * DKP + s;
      const float vj = live ? sv[tok * CPB + cl] : 0.f;
      float acc = 0.f;
      if (MODE == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          S[r] = fmaf(lam, S[r], kk[r * TPC] * vj);
          acc = fmaf(S[r], qk[r * TPC], acc);
        }
      } else {
        const float* gk = sg + (size_t)tok * DKP + s;
        float kr[R];
        float pred = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          kr[r] = kk[r * TPC];
          S[r] *= gk[r * TPC];
          pred = fmaf(S[r], kr[r], pred);
        }
        for (int o = TPC >> 1; o > 0; o >>= 1) pred += __shfl_xor_sync(L3_FULL, pred, o);
        const float u = sb[tok] * (vj - pred);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          S[r] = fmaf(kr[r], u, S[r]);
          acc = fmaf(S[r], qk[r * TPC], acc);
        }
      }
      for (int o = TPC >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(L3_FULL, acc, o);
      if (s == 0 && live) so[tok * CPB + cl] = acc;
    }
    __syncthreads();
    for (int idx = tid; idx < n * CPB; idx += nthr) {
      const int tok = idx / CPB, c = idx - tok * CPB;
      const int jj = tile * CPB + c;
      if (jj < a.DV) a.out[((size_t)b * a.L + t0 + tok) * ((size_t)a.H * a.DV) + (size_t)h * a.DV + jj] = so[idx];
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = s + r * TPC;
    if (col_ok && i < a.DK) Sg[(size_t)i * a.DV + j] = S[r];
  }
}

int pow2_at_least(int v) {
  int p = 1;
  while (p < v) p <<= 1;
  return p;
}

template <int R>
cudaError_t launch_recur_r(const RecurArgs& a, cudaStream_t s) {
  const int TPC = std::min(32, pow2_at_least((a.DK + R - 1) / R));
  const int CPB = std::max(1, std::min(256 / TPC, pow2_at_least(a.DV)));
  const int threads = std::max(32, CPB * TPC);  // CPB * TPC is a power of two: whole warps once it reaches 32
  const int DKP = R * TPC;
  const int per_tok = (a.mode == 1 ? 3 : 2) * DKP + 2 * CPB + 1;
  const int TCH = std::max(1, std::min(32, 11000 / per_tok));
  const size_t smem = (size_t)TCH * per_tok * sizeof(float);
  const int ntile = (a.DV + CPB - 1) / CPB;
  const dim3 grid(a.H * ntile, a.B);
  if (a.mode == 0) return launch_k(recur_kernel<R, 0>, grid, dim3(threads), smem, s, a, TPC, CPB, TCH);
  return launch_k(recur_kernel<R, 1>, grid, dim3(threads), smem, s, a, TPC, CPB, TCH);
}

}  // namespace

bool recur_supported(int DK, int DV) { return DK >= 1 && DK <= 1024 && DV >= 1; }

cudaError_t launch_recur(const RecurArgs& a, cudaStream_t s) {
  if (!recur_supported(a.DK, a.DV)) return cudaErrorInvalidValue;
  if (a.DK <= 256) return launch_recur_r<8>(a, s);
  return launch_recur_r<32>(a, s);
}
