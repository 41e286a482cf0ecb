// Causal softmax attention over the KV cache for head sizes the tiled kernels of attention.cu do not take
// (they are compiled for a list of head sizes that are multiples of 4): any HD, prompt rows and decode alike.
// One warp per (sequence, token, query head); a lane scores one key of a batch of 32, the batch's weights are
// then spread by shuffles while the lanes own output dimensions.  Scores, weights and sums are fp32.  Same
// argument struct and the same meaning of scale / head_gate as the tiled kernels.
#include "common.cuh"
#include "mixer.h"

namespace {

template <typename KVT>
__global__ void __launch_bounds__(128) attn_any_kernel(AttnArgs a) {
  extern __shared__ float sm[];  // per warp: q [HD] | o [HD]
  pdl_launch();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int item = blockIdx.x * 4 + warp;
  const int HD = a.HD;
  if (item >= a.B * a.L * a.HN) return;
  const int head = item % a.HN, row = item / a.HN;
  const int b = row / a.L, t = row - b * a.L;
  const int last = (a.row_pos ? a.row_pos[b] : *a.pos_ptr) + t;  // keys [0, last] are visible
  const int kvh = head / (a.HN / a.KVHN);
  float* q = sm + (size_t)warp * 2 * HD;
  float* o = q + HD;
  for (int d = lane; d < HD; d += 32) { q[d] = a.q[((size_t)row * a.HN + head) * HD + d]; o[d] = 0.f; }
  __syncwarp();
  const KVT* kb = (const KVT*)a.cache_k + ((size_t)b * a.KVHN + kvh) * a.M * HD;
  const KVT* vb = (const KVT*)a.cache_v + ((size_t)b * a.KVHN + kvh) * a.M * HD;
  const float scale = attn_scale(a, HD);
  float mx = -INFINITY, l = 0.f;
  for (int j0 = 0; j0 <= last; j0 += 32) {
    const int j = j0 + lane;
    float sc = -INFINITY;
    if (j <= last) {
      float d0 = 0.f;
      const KVT* kr = kb + (size_t)j * HD;
      for (int d = 0; d < HD; ++d) d0 = fmaf(q[d], to_f32(kr[d]), d0);
      sc = d0 * scale;
    }
    const float mnew = fmaxf(mx, warp_max(sc));
    const float p = j <= last ? expf(sc - mnew) : 0.f;
    const float alpha = expf(mx - mnew);  // first batch: exp(-inf) = 0 and o, l are 0
    l = l * alpha + warp_sum(p);
    mx = mnew;
    const int nb = min(32, last + 1 - j0);
    for (int d0 = 0; d0 < HD; d0 += 32) {  // every lane runs every round: the shuffles name the full warp
      const int d = d0 + lane;
      const bool ok = d < HD;
      float acc = ok ? o[d] * alpha : 0.f;
      for (int u = 0; u < nb; ++u) {
        const float pu = __shfl_sync(L3_FULL, p, u);
        if (ok) acc = fmaf(pu, to_f32(vb[(size_t)(j0 + u) * HD + d]), acc);
      }
      if (ok) o[d] = acc;
    }
  }
  const float inv = attn_gate(a, (size_t)row, head) / l;
  for (int d = lane; d < HD; d += 32) {
    const float v = o[d] * inv;
    const size_t oi = ((size_t)row * a.HN + head) * HD + d;
    if (a.out) a.out[oi] = v;
    if (a.out_bf16) a.out_bf16[oi] = __float2bfloat16_rn(v);
  }
}

}  // namespace

cudaError_t launch_attn_any(const AttnArgs& a, bool kv_bf16, cudaStream_t s) {
  const int items = a.B * a.L * a.HN;
  const size_t smem = (size_t)4 * 2 * a.HD * sizeof(float);
  const dim3 grid((items + 3) / 4);
  if (kv_bf16) return launch_k(attn_any_kernel<bf16>, grid, dim3(128), smem, s, a);
  return launch_k(attn_any_kernel<float>, grid, dim3(128), smem, s, a);
}
