// C-ABI of libllama3_b200.so (include/llama3_b200.h): model state in HBM, weight packing,
// orchestration of one forward step (Llama.__call__, llama3.py:285-308) and of the greedy
// loop (Llama.generate, llama3.py:310-321) as CUDA-graph replays with every per-step scalar
// (position, output column, next token ids) resident on the device.
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <string>
#include <vector>

#include "../../include/llama3_b200.h"
#include "common.cuh"
#include "gemm_tc.h"
#include "internal.h"
#include "layerlist.h"
#include "mega.h"
#include "model.h"
#include "stack.h"

static thread_local char g_err[512] = "";
const bool g_l3_debug_sync = getenv("L3_DEBUG_SYNC") && atoi(getenv("L3_DEBUG_SYNC")) != 0;
bool g_l3_pdl_next = false;  // one-shot: the next launch is a programmatic dependent of its predecessor (linear())
bool g_l3_pdl = false;  // programmatic dependent launch for step kernels (common.cuh); measured slower
                        // than plain graph edges on this workload, so opt-in (L3_PDL=1)

#include <mutex>
#include <set>
bool l3_carveout_seen(const void* fn) {
  static std::mutex mu;
  static std::set<std::pair<int, const void*>> seen;
  if (!getenv("L3_CARVEOUT")) return true;  // measured: a smaller L1 costs the streaming kernels more than it saves
  int dev = 0;
  cudaGetDevice(&dev);
  std::lock_guard<std::mutex> g(mu);
  return !seen.insert({dev, fn}).second;
}

void set_err(L3Model* m, const char* fmt, ...) {  // also used by packed_io.cu
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  snprintf(g_err, sizeof g_err, "%s", buf);
  if (m) snprintf(m->err, sizeof m->err, "%s", buf);
}

extern "C" const char* l3_version(void) { return "llama3_b200 0.1 (sm_100a)"; }
extern "C" const char* l3_last_error(const L3Model* m) { return m ? m->err : g_err; }
extern "C" int l3_device_count(int* out) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) { set_err(nullptr, "cudaGetDeviceCount: %s", cudaGetErrorString(e)); *out = 0; return L3_ECUDA; }
  *out = n;
  return L3_OK;
}

static size_t wbytes(const L3Model* m) { return m->bf16 ? 2 : 4; }

// ------------------------------------------------------------------------------ create
extern "C" int l3_create(const L3Config* c, L3Model** out) {
  *out = nullptr;
  REQUIRE(nullptr, c->dim > 0 && c->n_layers > 0 && c->n_heads > 0 && c->n_kv_heads > 0, "bad config");
  REQUIRE(nullptr, c->dim % c->n_heads == 0, "dim %d not divisible by n_heads %d", c->dim, c->n_heads);
  REQUIRE(nullptr, c->n_heads % c->n_kv_heads == 0, "n_heads %% n_kv_heads != 0 (llama3.py:127)");
  REQUIRE(nullptr, c->dim % 8 == 0 && c->hidden_dim % 8 == 0, "dim and hidden_dim must be multiples of 8");
  REQUIRE(nullptr, attn_head_dim_supported(c->dim / c->n_heads), "head_dim %d unsupported (16,32,48,64,96,128)",
          c->dim / c->n_heads);
  REQUIRE(nullptr, c->dtype == L3_DTYPE_F32 || c->dtype == L3_DTYPE_BF16, "bad dtype");
  REQUIRE(nullptr, c->tp_world >= 1 && c->tp_rank >= 0 && c->tp_rank < c->tp_world, "bad tp rank/world");
  REQUIRE(nullptr, c->n_kv_heads % c->tp_world == 0 && c->hidden_dim % (8 * c->tp_world) == 0 &&
                       c->vocab_size % c->tp_world == 0,
          "tensor parallel world %d must divide n_kv_heads, hidden_dim/8 and vocab_size", c->tp_world);
  REQUIRE(nullptr, c->tp_world <= L3_MAX_TP, "tensor parallel world %d exceeds %d", c->tp_world, L3_MAX_TP);
  REQUIRE(nullptr, c->max_batch_size >= 1 && c->max_seq_len >= 1 && c->vocab_size >= 1, "bad sizes");

  if (getenv("L3_PDL")) g_l3_pdl = atoi(getenv("L3_PDL")) != 0;
  if (c->flags & L3_FLAG_NO_PDL) g_l3_pdl = false;
  L3Model* m = new L3Model();
  m->cfg = *c;
  m->bf16 = c->dtype == L3_DTYPE_BF16;
  m->D = c->dim;
  m->HD = c->dim / c->n_heads;
  m->G = c->tp_world;
  m->HN = c->n_heads / m->G;
  m->KVHN = c->n_kv_heads / m->G;
  m->FD = c->hidden_dim / m->G;
  m->VS = c->vocab_size / m->G;
  m->M = c->max_seq_len;
  m->maxB = c->max_batch_size;
  m->qkv_rows = (m->HN + 2 * m->KVHN) * m->HD;
  if (cudaSetDevice(c->device) != cudaSuccess) {
    set_err(nullptr, "cudaSetDevice(%d) failed: %s", c->device, cudaGetErrorString(cudaGetLastError()));
    delete m;
    return L3_ECUDA;
  }
  cudaError_t e = cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) { set_err(nullptr, "stream: %s", cudaGetErrorString(e)); delete m; return L3_ECUDA; }
  cudaEventCreate(&m->ev0);
  cudaEventCreate(&m->ev1);

  const size_t wb = wbytes(m);
  auto alloc = [&](void** p, size_t bytes) { return cudaMalloc(p, bytes); };
#define AL(p, bytes)                                                                                  \
  if ((e = alloc((void**)&(p), (bytes))) != cudaSuccess) {                                            \
    set_err(nullptr, "cudaMalloc(%zu) failed: %s", (size_t)(bytes), cudaGetErrorString(e));           \
    l3_destroy(m);                                                                                    \
    return L3_ENOMEM;                                                                                 \
  }
  AL(m->embed, (size_t)c->vocab_size * m->D * wb);
  AL(m->lm_head, (size_t)m->VS * m->D * wb);
  AL(m->norm_final, (size_t)m->D * 4);
  m->layers.resize(c->n_layers);
  for (auto& L : m->layers) {
    AL(L.wqkv, (size_t)m->qkv_rows * m->D * wb);
    AL(L.wo, (size_t)m->D * m->HN * m->HD * wb);
    AL(L.w13, (size_t)2 * m->FD * m->D * wb);
    AL(L.w2, (size_t)m->D * m->FD * wb);
    AL(L.norm_in, (size_t)m->D * 4);
    AL(L.norm_post, (size_t)m->D * 4);
  }
  AL(m->cos_tab, (size_t)m->M * (m->HD / 2) * 4);
  AL(m->sin_tab, (size_t)m->M * (m->HD / 2) * 4);
#undef AL
  m->loaded.assign(3 + (size_t)c->n_layers * 9, 0);
  *out = m;
  return L3_OK;
}

extern "C" int l3_destroy(L3Model* m) {
  if (!m) return L3_OK;
  cudaSetDevice(m->cfg.device);
  if (m->stream) cudaStreamSynchronize(m->stream);
  // graphs first: NCCL keeps a reference per captured collective and ncclCommDestroy waits for them
  for (auto& g : m->graphs) {
    if (g.exec) cudaGraphExecDestroy(g.exec);
    if (g.graph) cudaGraphDestroy(g.graph);
  }
  m->graphs.clear();
  tp_destroy(m);
  ll_destroy(m);
  if (m->logits_loc) cudaFree(m->logits_loc);
  if (m->logits_all) cudaFree(m->logits_all);
  auto fr = [](void* p) { if (p) cudaFree(p); };
  fr(m->embed); fr(m->lm_head); fr(m->norm_final); fr(m->cos_tab); fr(m->sin_tab);
  for (auto& L : m->layers) {
    fr(L.wqkv); fr(L.wo); fr(L.w13); fr(L.w2); fr(L.norm_in); fr(L.norm_post); fr(L.ck); fr(L.cv);
    for (int i = 0; i < 4; ++i) { fr(L.w_hi[i]); fr(L.w_lo[i]); }
  }
  fr(m->xn_lo); fr(m->ctx_lo); fr(m->h_lo); fr(m->xlast_lo); fr(m->lm_hi); fr(m->lm_lo);
  fr(m->gemm_part); fr(m->gemm_cnt); fr(m->xn16); fr(m->ctx16); fr(m->h16); fr(m->xlast16); fr(m->q16);
  fr(m->stage); fr(m->x); fr(m->xn); fr(m->q); fr(m->ctx); fr(m->h); fr(m->xlast); fr(m->logits);
  fr(m->d_mega_layers); fr(m->d_mega_bar); fr(m->d_mega_ll); fr(m->d_mega_dbg);
  fr(m->d_stack_layers); fr(m->d_stack_dbg); fr(m->d_stack_dbgx);
  for (auto p : m->stack_wpack) fr(p);
  fr(m->d_rowlen); fr(m->d_rowpos); fr(m->d_done); fr(m->d_lastrow);
  fr(m->part_o); fr(m->part_ml); fr(m->attn_cnt); fr(m->d_ids); fr(m->d_fwd_ids); fr(m->d_next); fr(m->d_fwd_next); fr(m->d_scal); fr(m->d_tokens); fr(m->d_fwd_arg); fr(m->d_best); fr(m->l2buf);
  if (m->h_next) cudaFreeHost(m->h_next);
  if (m->ev0) cudaEventDestroy(m->ev0);
  if (m->ev1) cudaEventDestroy(m->ev1);
  if (m->stream) cudaStreamDestroy(m->stream);
  delete m;
  return L3_OK;
}

// ------------------------------------------------------------------------------ weights
struct KeyInfo { int layer; int kind; };  // kind: 0 embed 1 final norm 2 lm_head; 10.. per layer
enum { K_Q = 10, K_K, K_V, K_O, K_UP, K_GATE, K_DOWN, K_NIN, K_NPOST };

static bool parse_key(const char* key, KeyInfo* ki) {
  if (!strcmp(key, "model.embed_tokens.weight")) { *ki = {-1, 0}; return true; }
  if (!strcmp(key, "model.norm.weight")) { *ki = {-1, 1}; return true; }
  if (!strcmp(key, "lm_head.weight")) { *ki = {-1, 2}; return true; }
  int layer = -1, n = 0;
  if (sscanf(key, "model.layers.%d.%n", &layer, &n) < 1 || n == 0) return false;
  const char* rest = key + n;
  static const struct { const char* name; int kind; } tab[] = {
      {"self_attn.q_proj.weight", K_Q},        {"self_attn.k_proj.weight", K_K},
      {"self_attn.v_proj.weight", K_V},        {"self_attn.o_proj.weight", K_O},
      {"mlp.up_proj.weight", K_UP},            {"mlp.gate_proj.weight", K_GATE},
      {"mlp.down_proj.weight", K_DOWN},        {"input_layernorm.weight", K_NIN},
      {"post_attention_layernorm.weight", K_NPOST}};
  for (auto& t : tab)
    if (!strcmp(rest, t.name)) { *ki = {layer, t.kind}; return true; }
  return false;
}

// Where a logical tensor lands: destination matrix, which global rows/cols this rank keeps,
// and the row mapping inside the packed matrix.
struct Place {
  void* dst; bool is_norm;
  int64_t g_rows, g_cols;      // logical (global) shape
  int64_t row0, rows;          // slice of global rows kept by this rank
  int64_t col0, cols;          // slice of global cols kept
  int dst_row0, dst_row_stride, dst_ld;
  uint32_t tensor_id; float scale, bias;
};

static int place_of(L3Model* m, const KeyInfo& ki, Place* p) {
  const int D = m->D, HD = m->HD, r = m->cfg.tp_rank;
  const int gHN = m->cfg.n_heads, gKV = m->cfg.n_kv_heads, gFD = m->cfg.hidden_dim, gVS = m->cfg.vocab_size;
  *p = Place{};
  p->dst_row_stride = 1;
  p->bias = 0.f;
  p->tensor_id = (uint32_t)((ki.layer + 1) * 16 + ki.kind);
  auto lin = [&](int fan_in) { p->scale = 0.85f / sqrtf((float)fan_in); };
  if (ki.layer < 0) {
    if (ki.kind == 0) { *p = Place{m->embed, false, gVS, D, 0, gVS, 0, D, 0, 1, D, p->tensor_id, 0.5f, 0.f}; return 0; }
    if (ki.kind == 1) { *p = Place{m->norm_final, true, D, 1, 0, D, 0, 1, 0, 1, 1, p->tensor_id, 0.1f, 1.f}; return 0; }
    lin(D);
    *p = Place{m->lm_head, false, gVS, D, (int64_t)r * m->VS, m->VS, 0, D, 0, 1, D, p->tensor_id, p->scale, 0.f};
    return 0;
  }
  if (ki.layer >= m->cfg.n_layers) return -1;
  L3Layer& L = m->layers[ki.layer];
  switch (ki.kind) {
    case K_Q: lin(D); *p = Place{L.wqkv, false, (int64_t)gHN * HD, D, (int64_t)r * m->HN * HD, (int64_t)m->HN * HD, 0, D, 0, 1, D, p->tensor_id, p->scale, 0.f}; break;
    case K_K: lin(D); *p = Place{L.wqkv, false, (int64_t)gKV * HD, D, (int64_t)r * m->KVHN * HD, (int64_t)m->KVHN * HD, 0, D, m->HN * HD, 1, D, p->tensor_id, p->scale, 0.f}; break;
    case K_V: lin(D); *p = Place{L.wqkv, false, (int64_t)gKV * HD, D, (int64_t)r * m->KVHN * HD, (int64_t)m->KVHN * HD, 0, D, (m->HN + m->KVHN) * HD, 1, D, p->tensor_id, p->scale, 0.f}; break;
    case K_O: lin(gHN * HD); *p = Place{L.wo, false, D, (int64_t)gHN * HD, 0, D, (int64_t)r * m->HN * HD, (int64_t)m->HN * HD, 0, 1, m->HN * HD, p->tensor_id, p->scale, 0.f}; break;
    case K_GATE: lin(D); *p = Place{L.w13, false, gFD, D, (int64_t)r * m->FD, m->FD, 0, D, 0, 2, D, p->tensor_id, p->scale, 0.f}; break;
    case K_UP: lin(D); *p = Place{L.w13, false, gFD, D, (int64_t)r * m->FD, m->FD, 0, D, 1, 2, D, p->tensor_id, p->scale, 0.f}; break;
    case K_DOWN: lin(gFD); *p = Place{L.w2, false, D, gFD, 0, D, (int64_t)r * m->FD, m->FD, 0, 1, m->FD, p->tensor_id, p->scale, 0.f}; break;
    case K_NIN: *p = Place{L.norm_in, true, D, 1, 0, D, 0, 1, 0, 1, 1, p->tensor_id, 0.1f, 1.f}; break;
    case K_NPOST: *p = Place{L.norm_post, true, D, 1, 0, D, 0, 1, 0, 1, 1, p->tensor_id, 0.1f, 1.f}; break;
    default: return -1;
  }
  return 0;
}

static size_t loaded_slot(const KeyInfo& ki) { return ki.layer < 0 ? (size_t)ki.kind : 3 + (size_t)ki.layer * 9 + (ki.kind - 10); }

extern "C" int l3_load_weight(L3Model* m, const char* key, const float* host, const int64_t* shape, int ndim) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, !m->ll, "a layer-list handle takes its tensors through l3_load_tensor");
  REQUIRE(m, !m->finalized, "l3_load_weight after l3_finalize");
  CK(m, cudaSetDevice(m->cfg.device));
  KeyInfo ki;
  REQUIRE(m, parse_key(key, &ki), "unknown weight key '%s'", key);
  Place p;
  REQUIRE(m, place_of(m, ki, &p) == 0, "layer index out of range in '%s'", key);
  REQUIRE(m, ndim == 1 || ndim == 2, "'%s': expected a vector or a matrix, got %d dimensions", key, ndim);
  const int64_t rows = shape[0], cols = ndim > 1 ? shape[1] : 1;
  REQUIRE(m, rows == p.g_rows && cols == p.g_cols,
          "shape mismatch for '%s': got [%lld, %lld], want [%lld, %lld]", key, (long long)rows, (long long)cols,
          (long long)p.g_rows, (long long)p.g_cols);
  // stage row chunks of the kept slice as fp32, then pack/convert on the device
  const size_t STAGE = (size_t)256 << 20;
  if (!m->stage) CK(m, cudaMalloc((void**)&m->stage, STAGE));
  const int64_t rows_per = std::max<int64_t>(1, (int64_t)(STAGE / (p.cols * sizeof(float))));
  for (int64_t r0 = 0; r0 < p.rows; r0 += rows_per) {
    const int64_t nr = std::min(rows_per, p.rows - r0);
    const float* src = host + (p.row0 + r0) * p.g_cols + p.col0;
    CK(m, cudaMemcpy2DAsync(m->stage, p.cols * sizeof(float), src, p.g_cols * sizeof(float), p.cols * sizeof(float),
                            nr, cudaMemcpyHostToDevice, m->stream));
    CK(m, launch_pack_rows(m->stage, (int)nr, (int)p.cols, p.dst, p.is_norm ? false : m->bf16,
                           p.dst_row0 + (int)r0 * p.dst_row_stride, p.dst_row_stride, p.dst_ld, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));  // host buffer may be pageable and the stage is reused
  }
  m->loaded[loaded_slot(ki)] = 1;
  return L3_OK;
}

extern "C" int l3_fill_random(L3Model* m, uint64_t seed) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, !m->finalized, "l3_fill_random after l3_finalize");
  CK(m, cudaSetDevice(m->cfg.device));
  if (m->ll) return ll_fill_random(m, seed);
  std::vector<KeyInfo> keys = {{-1, 0}, {-1, 1}, {-1, 2}};
  for (int l = 0; l < m->cfg.n_layers; ++l)
    for (int k = K_Q; k <= K_NPOST; ++k) keys.push_back({l, k});
  for (auto& ki : keys) {
    Place p;
    place_of(m, ki, &p);
    CK(m, launch_fill_random(p.dst, p.is_norm ? false : m->bf16, p.rows, p.cols, p.g_cols, p.row0, p.col0, p.dst_row0,
                             p.dst_row_stride, p.dst_ld, seed, p.tensor_id, p.scale, p.bias, m->stream));
    m->loaded[loaded_slot(ki)] = 1;
  }
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

extern "C" int l3_set_rope_tables(L3Model* m, const double* cos_tab, const double* sin_tab) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, !m->ll, "layer-list handles have no rotary tables");
  CK(m, cudaSetDevice(m->cfg.device));
  const size_t n = (size_t)m->M * (m->HD / 2);
  std::vector<float> c(n), s(n);
  for (size_t i = 0; i < n; ++i) { c[i] = (float)cos_tab[i]; s[i] = (float)sin_tab[i]; }
  CK(m, cudaMemcpy(m->cos_tab, c.data(), n * 4, cudaMemcpyHostToDevice));
  CK(m, cudaMemcpy(m->sin_tab, s.data(), n * 4, cudaMemcpyHostToDevice));
  m->rope_set = true;
  return L3_OK;
}

extern "C" int l3_finalize(L3Model* m) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, !m->finalized, "already finalized");
  CK(m, cudaSetDevice(m->cfg.device));
  if (m->ll) return ll_finalize(m);
  for (size_t i = 0; i < m->loaded.size(); ++i)
    if (!m->loaded[i]) { set_err(m, "weight slot %zu was never loaded", i); return L3_ESTATE; }
  if (!m->rope_set) { set_err(m, "l3_set_rope_tables was not called"); return L3_ESTATE; }
  if (m->stage) { cudaFree(m->stage); m->stage = nullptr; }

  const size_t kvb = m->bf16 ? 2 : 4;
  const size_t cache_bytes = (size_t)m->maxB * m->KVHN * m->M * m->HD * kvb;
  for (auto& L : m->layers) {
    CK(m, cudaMalloc(&L.ck, cache_bytes));
    CK(m, cudaMalloc(&L.cv, cache_bytes));
    CK(m, cudaMemsetAsync(L.ck, 0, cache_bytes, m->stream));  // np.zeros, llama3.py:138-153
    CK(m, cudaMemsetAsync(L.cv, 0, cache_bytes, m->stream));
  }
  // activation workspace: rows of one chunk (long prompts are processed in chunks, which the
  // reference's mask construction defines exactly: llama3.py:293-297 with start_pos > 0)
  const int64_t want = (int64_t)m->maxB * m->M;
  m->cap_tok = (int)std::max<int64_t>(m->maxB, std::min<int64_t>(want, 8192));
  const size_t ct = (size_t)m->cap_tok;
  CK(m, cudaMalloc((void**)&m->x, ct * m->D * 4));
  CK(m, cudaMalloc((void**)&m->xn, ct * m->D * 4));
  CK(m, cudaMalloc((void**)&m->q, ct * m->HN * m->HD * 4));
  CK(m, cudaMalloc((void**)&m->ctx, ct * m->HN * m->HD * 4));
  CK(m, cudaMalloc((void**)&m->h, ct * m->FD * 4));
  CK(m, cudaMalloc((void**)&m->xlast, (size_t)m->maxB * m->D * 4));
  CK(m, cudaMalloc((void**)&m->logits, (size_t)m->maxB * m->cfg.vocab_size * 4));
  if (m->G > 1) {  // vocabulary-sharded LM head: local slice, and the all-gathered slices of every rank
    CK(m, cudaMalloc((void**)&m->logits_loc, (size_t)m->maxB * m->VS * 4));
    CK(m, cudaMalloc((void**)&m->logits_all, (size_t)m->G * m->maxB * m->VS * 4));
  }
  m->tc_ok = !(m->cfg.flags & L3_FLAG_NO_TENSORCORE) && tc_gemm_supported(m->D) && tc_gemm_supported(m->FD);
  if (m->tc_ok && !(getenv("L3_GEMM_KSPLIT") && atoi(getenv("L3_GEMM_KSPLIT")) == 0)) {
    CK(m, cudaMalloc((void**)&m->gemm_part, (size_t)32 << 20));
    CK(m, cudaMalloc((void**)&m->gemm_cnt, 1024 * sizeof(int)));
    CK(m, cudaMemsetAsync(m->gemm_cnt, 0, 1024 * sizeof(int), m->stream));
  }
  if (m->tc_ok && !m->bf16) {
    CK(m, cudaMalloc((void**)&m->xn_lo, ct * m->D * 4));
    CK(m, cudaMalloc((void**)&m->ctx_lo, ct * m->HN * m->HD * 4));
    CK(m, cudaMalloc((void**)&m->h_lo, ct * m->FD * 4));
    CK(m, cudaMalloc((void**)&m->xlast_lo, (size_t)m->maxB * m->D * 4));
    auto split = [&](const void* src, size_t n, float** hi, float** lo) -> int {
      CK(m, cudaMalloc((void**)hi, n * 4));
      CK(m, cudaMalloc((void**)lo, n * 4));
      CK(m, launch_split_tf32((const float*)src, *hi, *lo, (int64_t)n, m->stream));
      return L3_OK;
    };
    int rc;
    for (auto& L : m->layers) {
      if ((rc = split(L.wqkv, (size_t)m->qkv_rows * m->D, &L.w_hi[0], &L.w_lo[0])) != L3_OK) return rc;
      if ((rc = split(L.wo, (size_t)m->D * m->HN * m->HD, &L.w_hi[1], &L.w_lo[1])) != L3_OK) return rc;
      if ((rc = split(L.w13, (size_t)2 * m->FD * m->D, &L.w_hi[2], &L.w_lo[2])) != L3_OK) return rc;
      if ((rc = split(L.w2, (size_t)m->D * m->FD, &L.w_hi[3], &L.w_lo[3])) != L3_OK) return rc;
    }
    if ((rc = split(m->lm_head, (size_t)m->VS * m->D, &m->lm_hi, &m->lm_lo)) != L3_OK) return rc;
  }
  if (m->tc_ok && m->bf16) {
    CK(m, cudaMalloc(&m->xn16, ct * m->D * 2));
    CK(m, cudaMalloc(&m->ctx16, ct * m->HN * m->HD * 2));
    CK(m, cudaMalloc(&m->h16, ct * m->FD * 2));
    CK(m, cudaMalloc(&m->xlast16, (size_t)m->maxB * m->D * 2));
    const char* env = getenv("L3_ATTN_TC");
    m->attn_tc_ok = attn_prefill_tc_supported(m->HD) && !(env && atoi(env) == 0);
    if (m->attn_tc_ok) CK(m, cudaMalloc(&m->q16, ct * m->HN * m->HD * 2));
  }
  m->max_split = 32;
  CK(m, cudaMalloc((void**)&m->part_o, (size_t)m->maxB * m->HN * m->max_split * m->HD * 4));
  CK(m, cudaMalloc((void**)&m->part_ml, (size_t)m->maxB * m->HN * m->max_split * 2 * 4));
  CK(m, cudaMalloc((void**)&m->attn_cnt, (size_t)m->maxB * m->HN * 4));
  CK(m, cudaMemsetAsync(m->attn_cnt, 0, (size_t)m->maxB * m->HN * 4, m->stream));
  CK(m, cudaMalloc((void**)&m->d_ids, (size_t)m->maxB * m->M * 4));
  CK(m, cudaMalloc((void**)&m->d_next, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_fwd_next, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_fwd_ids, (size_t)m->maxB * m->M * 4));
  CK(m, cudaMalloc((void**)&m->d_scal, 16 * 4));
  CK(m, cudaMemsetAsync(m->d_scal, 0, 16 * 4, m->stream));
  CK(m, cudaMalloc((void**)&m->d_tokens, (size_t)m->maxB * m->M * 8));
  CK(m, cudaMalloc((void**)&m->d_fwd_arg, (size_t)m->maxB * 8));
  CK(m, cudaMalloc((void**)&m->d_best, (size_t)m->maxB * 8));
  CK(m, cudaMemsetAsync(m->d_best, 0, (size_t)m->maxB * 8, m->stream));
  CK(m, cudaMallocHost((void**)&m->h_next, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_rowlen, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_rowpos, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_done, (size_t)m->maxB * 4));
  CK(m, cudaMalloc((void**)&m->d_lastrow, (size_t)m->maxB * 4));
  {  // persistent batch-1 decode kernel: per-layer pointer table + grid barrier state
    cudaDeviceProp prop;
    CK(m, cudaGetDeviceProperties(&prop, m->cfg.device));
    m->n_sm = prop.multiProcessorCount;
    const char* env = getenv("L3_MEGA");
    m->mega_ok = !(env && atoi(env) == 0) && !(m->cfg.flags & L3_FLAG_NO_MEGA) &&
                 decode_mega_supported(m->D, m->HN, m->KVHN, m->HD, m->FD, m->VS);
    if (m->mega_ok) {
      std::vector<MegaLayer> hl;
      for (auto& L : m->layers) hl.push_back(MegaLayer{L.wqkv, L.wo, L.w13, L.w2, L.norm_in, L.norm_post, L.ck, L.cv});
      CK(m, cudaMalloc(&m->d_mega_layers, hl.size() * sizeof(MegaLayer)));
      CK(m, cudaMemcpy(m->d_mega_layers, hl.data(), hl.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice));
      CK(m, cudaMalloc((void**)&m->d_mega_bar, 64));
      CK(m, cudaMemset(m->d_mega_bar, 0, 64));
      const size_t llw = (size_t)2 * L3_LL_WORDS + (size_t)m->HN * m->HD + (size_t)2 * L3_LL_VEC;
      CK(m, cudaMalloc((void**)&m->d_mega_ll, llw * 8));
      CK(m, cudaMemset(m->d_mega_ll, 0, llw * 8));  // tag 0 = "never written": exchange numbers start at 1
      if (getenv("L3_MEGA_DBG") && atoi(getenv("L3_MEGA_DBG"))) {
        CK(m, cudaMalloc((void**)&m->d_mega_dbg, (size_t)m->n_sm * 512 * 8));
        CK(m, cudaMemset(m->d_mega_dbg, 0, (size_t)m->n_sm * 512 * 8));
      }
    }
  }
  {  // cluster-resident batched decode (fp32, many sequences of a small model): packed per-CTA weight slabs
    const char* env = getenv("L3_STACK");
    const char* envb = getenv("L3_STACK_MIN_B");
    m->stack_min_B = envb ? atoi(envb) : 33;
    m->stack_ok = !(env && atoi(env) == 0) && !(m->cfg.flags & L3_FLAG_NO_MEGA) && m->G == 1 && !m->bf16 && m->tc_ok &&
                  m->maxB >= m->stack_min_B && decode_stack_supported(m->D, m->HN, m->KVHN, m->HD, m->FD, m->M) &&
                  decode_stack_max_clusters() > 0;
    if (m->stack_ok) {
      std::vector<StackLayer> hl;
      for (auto& L : m->layers) {
        float* wp = nullptr;
        CK(m, cudaMalloc((void**)&wp, decode_stack_pack_bytes(m->D, m->HN, m->HD, m->FD)));
        m->stack_wpack.push_back(wp);
        CK(m, decode_stack_pack_layer((const float*)L.wqkv, (const float*)L.wo, (const float*)L.w13, (const float*)L.w2, m->D,
                                      m->HN, m->HD, m->FD, wp, m->stream));
        hl.push_back(StackLayer{wp, L.norm_in, L.norm_post, (float*)L.ck, (float*)L.cv});
      }
      CK(m, cudaMalloc(&m->d_stack_layers, hl.size() * sizeof(StackLayer)));
      CK(m, cudaMemcpy(m->d_stack_layers, hl.data(), hl.size() * sizeof(StackLayer), cudaMemcpyHostToDevice));
      if (getenv("L3_STACK_DBG") && atoi(getenv("L3_STACK_DBG"))) {
        const size_t n = (size_t)((m->maxB + decode_stack_seqs_per_cluster() - 1) / decode_stack_seqs_per_cluster()) * 8 * 128;
        CK(m, cudaMalloc((void**)&m->d_stack_dbg, n * 8));
        CK(m, cudaMemset(m->d_stack_dbg, 0, n * 8));
        CK(m, cudaMalloc((void**)&m->d_stack_dbgx, (size_t)m->cfg.n_layers * 4 * m->maxB * m->D * 4));
        CK(m, cudaMemset(m->d_stack_dbgx, 0, (size_t)m->cfg.n_layers * 4 * m->maxB * m->D * 4));
      }
    }
  }
  CK(m, cudaStreamSynchronize(m->stream));
  // tensor parallel: ranks finish loading seconds apart; nobody pushes into a peer's receive area, or starts
  // waiting for a peer's flag, before every rank is here
  if (m->comm) { const int rc = tp_barrier(m); if (rc != L3_OK) return rc; }
  m->finalized = true;
  return L3_OK;
}

extern "C" int l3_reset_cache(L3Model* m) {
  if (!m || !m->finalized) return L3_ESTATE;
  CK(m, cudaSetDevice(m->cfg.device));
  if (m->ll) {
    const int rc = ll_reset_slots(m, 0, m->maxB, true);
    if (rc != L3_OK) return rc;
    CK(m, cudaStreamSynchronize(m->stream));
    return L3_OK;
  }
  const size_t cache_bytes = (size_t)m->maxB * m->KVHN * m->M * m->HD * (m->bf16 ? 2 : 4);
  for (auto& L : m->layers) {
    CK(m, cudaMemsetAsync(L.ck, 0, cache_bytes, m->stream));
    CK(m, cudaMemsetAsync(L.cv, 0, cache_bytes, m->stream));
  }
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

extern "C" int l3_read_cache(L3Model* m, int layer, float* k_out, float* v_out) {
  if (!m || !m->finalized) return L3_ESTATE;
  REQUIRE(m, layer >= 0 && layer < (m->ll ? (int)m->ll->runs.size() : m->cfg.n_layers), "layer out of range");
  CK(m, cudaSetDevice(m->cfg.device));
  if (m->ll) {  // a softmax layer run of a layer-list handle: its own head count and size
    const LLLayer& Ly = m->ll->layers[m->ll->runs[layer].layer];
    const LLState& St = m->ll->state[layer];
    REQUIRE(m, Ly.spec.mixer == L3_MIX_SOFTMAX, "layer %d keeps a recurrent state, not a KV cache (l3_read_state)", layer);
    const int G = Ly.spec.kv_heads, HD = Ly.spec.dim;
    const size_t n = (size_t)m->maxB * G * m->M * HD;
    float* tmp = nullptr;
    CK(m, cudaMalloc((void**)&tmp, n * 4));
    for (int which = 0; which < 2; ++which) {
      float* dst = which ? v_out : k_out;
      if (!dst) continue;
      CK(m, launch_cache_to_ref_layout(which ? St.cv : St.ck, m->bf16, m->maxB, G, m->M, HD, tmp, m->stream));
      CK(m, cudaMemcpyAsync(dst, tmp, n * 4, cudaMemcpyDeviceToHost, m->stream));
      CK(m, cudaStreamSynchronize(m->stream));
    }
    cudaFree(tmp);
    return L3_OK;
  }
  const size_t n = (size_t)m->maxB * m->KVHN * m->M * m->HD;
  float* tmp = nullptr;
  CK(m, cudaMalloc((void**)&tmp, n * 4));
  for (int which = 0; which < 2; ++which) {
    float* dst = which ? v_out : k_out;
    if (!dst) continue;
    CK(m, launch_cache_to_ref_layout(which ? m->layers[layer].cv : m->layers[layer].ck, m->bf16, m->maxB, m->KVHN,
                                     m->M, m->HD, tmp, m->stream));
    CK(m, cudaMemcpyAsync(dst, tmp, n * 4, cudaMemcpyDeviceToHost, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
  }
  cudaFree(tmp);
  return L3_OK;
}

// ------------------------------------------------------------------------------ one step
static int pick_nsplit(const L3Model* m, int B) {
  // Decode attention is latency-bound per CTA (a chain of dependent DRAM round trips: q, key batches, partial
  // publish, last-arriver combine), so what matters is that every CTA of the launch is resident at once: the keys of
  // a (sequence, kv head) are spread over as many CTAs as ONE wave holds at four CTAs of 128 threads per SM (the GQA
  // kernels are capped at 128 registers for that), as long as a split still sees >= 16 keys of the longest context.
  // Measured at 8B, batch 32 (ms per decode step; attention was 40 us of a 170 us layer with 5 splits = 3 waves):
  // 5 splits 5.57 (3 CTAs / SM) / 5.41 (4 CTAs / SM), 3 splits 5.29, 2 splits = one wave 4.99, 1 split 5.31.
  // The tensor-core kernel (bf16 GQA groups, attention.cu) does a CTA's keys in a fraction of the time, so there the
  // partial publish + last-arriver combine of a split costs more than it saves once every SM has a CTA: 256 CTAs.
  const int groups = B * m->KVHN;
  static const int target_env = [] { const char* v = getenv("L3_ATTN_TARGET_CTAS"); return v ? atoi(v) : 0; }();
  const int target = target_env > 0 ? target_env : attn_decode_mma_eligible(m->HD, m->HN / m->KVHN, m->bf16) ? 256 : 4 * 148;
  int ns = std::max(1, target / groups);
  const int by_len = std::max(1, m->M / 16);
  ns = std::min(std::min(ns, by_len), m->max_split);
  return std::max(ns, 1);
}

// Which activation buffer feeds a projection (decides where its GEMM-ready operand lives).
enum Feed { FEED_X_NORM, FEED_CTX, FEED_H, FEED_LAST_NORM };

// One projection y = f(x) @ W^T + epilogue.  Rows <= 8: row-streaming GEMV with the RMSNorm
// fused into its input staging.  More rows: tcgen05 tensor-core GEMM (bf16, or 3xTF32 in fp32
// mode) fed by operands its producer already wrote in GEMM-ready form; SIMT GEMM if the
// tensor-core path is switched off.
static int linear(L3Model* m, LinearArgs& a, Feed feed, const float* w_hi, const float* w_lo) {
  if (linear_rows_supported(a.rows, a.K)) {
    LAUNCH(m, launch_linear_rows(a, m->bf16, m->bf16, m->stream));
    return L3_OK;
  }
  const bool tc = m->tc_ok;
  const bool norm = a.norm_w != nullptr;
  float* n32 = feed == FEED_LAST_NORM ? m->xlast : m->xn;
  float* n32_lo = feed == FEED_LAST_NORM ? m->xlast_lo : m->xn_lo;
  void* n16 = feed == FEED_LAST_NORM ? m->xlast16 : m->xn16;
  if (norm) {  // the GEMM paths keep RMSNorm as its own pass, emitting the GEMM operand directly
    if (tc && m->bf16)
      LAUNCH(m, launch_rmsnorm(a.x, a.norm_w, a.eps, a.rows, a.K, a.src_mul, a.src_add, nullptr, (bf16*)n16, nullptr, m->stream, a.src_rows));
    else
      LAUNCH(m, launch_rmsnorm(a.x, a.norm_w, a.eps, a.rows, a.K, a.src_mul, a.src_add, n32, nullptr, tc ? n32_lo : nullptr, m->stream, a.src_rows));
    a.x = n32;
    a.src_rows = nullptr;
    a.norm_w = nullptr;
    a.src_mul = 1;
    a.src_add = 0;
  }
  if (!tc) {
    LAUNCH(m, launch_linear_simt(a, m->bf16, m->bf16, m->stream));
    return L3_OK;
  }
  TcGemmArgs t{};
  t.rows = a.rows; t.N = a.N; t.K = a.K; t.epi = a.epi; t.e = a.e; t.bn = 0;
  t.part = m->gemm_part; t.part_bytes = (size_t)32 << 20; t.tile_cnt = m->gemm_cnt; t.tile_cnt_len = 1024;
  if (m->bf16) {
    t.kind = TC_BF16;
    t.A[0] = feed == FEED_CTX ? m->ctx16 : feed == FEED_H ? m->h16 : n16;
    t.W[0] = a.W;
  } else {
    // LM head (rows >> tiles' K): one main accumulator is enough for K <= 512 and halves the TMEM columns
    // (an MMA costs 128 cycles whatever its width, so the LM head wants 256-wide tiles; L3_LM_2ACC=0 restores the
    // four-accumulator 64-wide tiles)
    static const bool lm2 = !(getenv("L3_LM_2ACC") && atoi(getenv("L3_LM_2ACC")) == 0);
    t.kind = (lm2 && feed == FEED_LAST_NORM && a.K <= 512 && (a.epi == EPI_ARGMAX || a.epi == EPI_STORE)) ? TC_TF32X3_2 : TC_TF32X3;
    t.A[0] = feed == FEED_CTX ? m->ctx : feed == FEED_H ? m->h : n32;
    t.A[1] = feed == FEED_CTX ? m->ctx_lo : feed == FEED_H ? m->h_lo : n32_lo;
    t.W[0] = w_hi;
    t.W[1] = w_lo;
  }
  static const bool swap_on = !(getenv("L3_GEMM_SWAP") && atoi(getenv("L3_GEMM_SWAP")) == 0);
  // Decode-sized batches: every swapped-role GEMM is launched as a programmatic dependent of whatever precedes it
  // (RMSNorm, attention, the previous GEMM), so that its prologue - TMEM allocation, barriers, tensor-map prefetch, the
  // first weight stage - runs under the predecessor's tail.  Measured at the 8B shape, ms per decode step at 32 rows:
  // off 4.34, behind RMSNorm only 4.27, every GEMM 4.17; at 128 rows (a 128-token prefill) it costs 6 %, and on every
  // kernel of the step (L3_PDL=1) it loses, so: these launches only.  L3_PDL_GEMM: 0 off, 1 behind RMSNorm, 2 all.
  static const int pdl_gemm = [] { const char* v = getenv("L3_PDL_GEMM"); return v ? atoi(v) : 2; }();
  if (swap_on && gemm_swap_supported(a.rows, a.N)) {  // 9..128 rows: weights as the 128-row operand
    g_l3_pdl_next = ((norm && pdl_gemm == 1) || pdl_gemm == 2) && a.rows <= 32 && !(m->cfg.flags & L3_FLAG_NO_PDL);
    const cudaError_t le = launch_gemm_swap(t, m->stream);
    g_l3_pdl_next = false;  // consumed by the launch; never left set for somebody else's kernel if the launcher bailed out
    LAUNCH(m, le);
  }
  else
    LAUNCH(m, launch_gemm_tc(t, m->stream));
  return L3_OK;
}

// where a step's argmax goes: int64 table (row stride, column from *step_ptr) and the int32 ids the NEXT step reads.
// The forward entry points use their own pair, so a forward call between two generate steps cannot disturb the loop.
struct OutSpec { int64_t* out64; int stride; const int* step_ptr; int32_t* next; };
// Ragged batch context of one chunk (null = every sequence shares start_pos and length):
// prefill: row_len (padding predicate) + last_rows (LM-head source rows); decode: row_pos.
struct Ragged { const int* row_pos; const int* row_len; const int32_t* last_rows; };

// Row-parallel projection under tensor parallelism (Wo, Wdown): this rank's partial product goes
// to the scratch rows in xn (dead at both call sites) - rank 0 folds the residual x into its
// partial - and the sum over ranks lands in x on every rank (tp_allreduce_sum, comm.cu).
static void tp_partial(L3Model* m, LinearArgs& a) {
  a.e.out = m->xn;
  if (m->cfg.tp_rank != 0) { a.epi = EPI_STORE; a.e.resid = nullptr; }
}

// A row-parallel projection (Wo, Wdown) with its residual add, on one GPU or summed over the
// tensor-parallel ranks.  Messages up to 64 Ki floats take the one-shot peer-memory exchange, larger
// ones NCCL; in bf16 mode the large partials travel as bf16 (half the NVLink bytes) and are added to
// the fp32 residual stream afterwards.
static int tp_row_parallel(L3Model* m, LinearArgs& a, Feed feed, const float* w_hi, const float* w_lo, int ntok, bool tc_rows) {
  int rc;
  if (m->G == 1) return linear(m, a, feed, w_hi, w_lo);
  const int64_t count = (int64_t)ntok * m->D;
  static const bool bf16_ar = !(getenv("L3_TP_BF16_AR") && atoi(getenv("L3_TP_BF16_AR")) == 0);
  if (bf16_ar && m->bf16 && tc_rows && m->xn16 && count > L3_LL2_WORDS && count % 8 == 0) {
    a.epi = EPI_STORE; a.e.out = nullptr; a.e.resid = nullptr; a.e.out_bf16 = (bf16*)m->xn16;
    if ((rc = linear(m, a, feed, w_hi, w_lo)) != L3_OK) return rc;
    if ((rc = tp_allreduce_sum_bf16(m, m->xn16, count)) != L3_OK) return rc;
    LAUNCH(m, launch_add_bf16(m->x, (const bf16*)m->xn16, count, m->stream));
    return L3_OK;
  }
  tp_partial(m, a);
  if ((rc = linear(m, a, feed, w_hi, w_lo)) != L3_OK) return rc;
  return tp_allreduce_sum(m, m->xn, m->x, count);
}

// Enqueue one chunk: tokens ids[b * ids_ld + ids_off + t], t < L, at start_pos = *d_pos.
// Layer-list handles: d_rows / n_rows choose the rows whose logits are wanted (null: the last token of every sequence),
// d_resid (may be null) receives the residual stream after every layer.
static int enqueue_chunk(L3Model* m, const int32_t* d_ids, int ids_ld, int ids_off, int B, int L, bool want_logits,
                         bool want_argmax, OutSpec os, const Ragged* rg = nullptr, const int32_t* d_rows = nullptr,
                         int n_rows = 0, float* d_resid = nullptr) {
  const int ntok = B * L, D = m->D, HD = m->HD;
  if (m->ll) {
    LAUNCH(m, launch_embed(m->embed, m->bf16, d_ids, ids_ld, ids_off, L, ntok, D, m->cfg.vocab_size, m->x, m->stream));
    int rc = ll_enqueue_layers(m, d_ids, ids_ld, ids_off, B, L, d_resid);
    if (rc != L3_OK) return rc;
    if (want_logits || want_argmax) {
      if ((rc = ll_enqueue_head(m, B, L, d_rows, n_rows)) != L3_OK) return rc;
      if (want_argmax) LAUNCH(m, launch_argmax(m->logits, B, m->VS, os.next, os.out64, os.stride, os.step_ptr, m->stream));
    }
    return L3_OK;
  }
  int* d_pos = m->d_scal + 0;
  // do this chunk's projections run as tensor-core GEMMs?  (their producers then write operands)
  const bool tc_rows = m->tc_ok && !linear_rows_supported(ntok, D);
  const bool tc_h = m->tc_ok && !linear_rows_supported(ntok, m->FD);
  const bool tc_ctx = m->tc_ok && !linear_rows_supported(ntok, m->HN * HD);
  LAUNCH(m, launch_embed(m->embed, m->bf16, d_ids, ids_ld, ids_off, L, ntok, D, m->cfg.vocab_size, m->x, m->stream));
  EpiArgs base{};
  base.cos_tab = m->cos_tab; base.sin_tab = m->sin_tab; base.pos_ptr = d_pos;
  base.L = L; base.HD = HD; base.HN = m->HN; base.KVHN = m->KVHN; base.M = m->M;
  if (rg) { base.row_pos = rg->row_pos; base.row_len = rg->row_len; }
  int rc;
  for (auto& Ly : m->layers) {
    LinearArgs a{};
    // q, k, v = rope(norm(x) @ Wqkv^T); k, v -> cache            llama3.py:248, 166-187
    a.W = Ly.wqkv; a.x = m->x; a.rows = ntok; a.N = m->qkv_rows; a.K = D;
    a.norm_w = Ly.norm_in; a.eps = m->cfg.norm_eps; a.src_mul = 1; a.src_add = 0;
    a.epi = EPI_ROPE_KV; a.e = base; a.e.out = m->q; a.e.ld_out = m->HN * HD;
    a.e.cache_k = Ly.ck; a.e.cache_v = Ly.cv;
    // bf16 prefill of more than 8 rows: tensor-core flash attention reads q as a bf16 TMA operand
    const bool attn_tc = L > 1 && tc_rows && tc_ctx && m->bf16 && m->attn_tc_ok;
    if (attn_tc) { a.e.out = nullptr; a.e.out_bf16 = (bf16*)m->q16; }
    if ((rc = linear(m, a, FEED_X_NORM, Ly.w_hi[0], Ly.w_lo[0])) != L3_OK) return rc;
    // ctx = softmax(q k^T / sqrt(HD) + mask) v                    llama3.py:190-207
    AttnArgs at{};
    at.q = m->q; at.cache_k = Ly.ck; at.cache_v = Ly.cv; at.pos_ptr = d_pos;
    at.row_pos = rg ? rg->row_pos : nullptr;
    at.B = B; at.L = L; at.HN = m->HN; at.KVHN = m->KVHN; at.HD = HD; at.M = m->M;
    at.part_o = m->part_o; at.part_ml = m->part_ml; at.counters = m->attn_cnt;
    if (tc_ctx && m->bf16) at.out_bf16 = (bf16*)m->ctx16;
    else { at.out = m->ctx; at.out_lo = tc_ctx ? m->ctx_lo : nullptr; }
    if (L == 1) {
      at.nsplit = pick_nsplit(m, B);
      LAUNCH(m, launch_attn_decode(at, m->bf16, m->stream));
    } else if (attn_tc) {
      at.nsplit = 1;
      at.cache_rows = m->maxB * m->KVHN * m->M;
      LAUNCH(m, launch_attn_prefill_tc(at, (const bf16*)m->q16, m->stream));
    } else {
      at.nsplit = 1;
      LAUNCH(m, launch_attn_prefill(at, m->bf16, m->stream));
    }
    // x = x + ctx @ Wo^T                                          llama3.py:210-211, 253
    a = LinearArgs{};
    a.W = Ly.wo; a.x = m->ctx; a.rows = ntok; a.N = D; a.K = m->HN * HD; a.src_mul = 1;
    a.epi = EPI_RESID; a.e = base; a.e.out = m->x; a.e.resid = m->x; a.e.ld_out = D;
    if ((rc = tp_row_parallel(m, a, FEED_CTX, Ly.w_hi[1], Ly.w_lo[1], ntok, tc_rows)) != L3_OK) return rc;
    // h = silu(norm(x) @ Wgate^T) * (norm(x) @ Wup^T)             llama3.py:256, 99-101
    a = LinearArgs{};
    a.W = Ly.w13; a.x = m->x; a.rows = ntok; a.N = 2 * m->FD; a.K = D;
    a.norm_w = Ly.norm_post; a.eps = m->cfg.norm_eps; a.src_mul = 1;
    a.epi = EPI_SWIGLU; a.e = base; a.e.ld_out = m->FD;
    if (tc_h && m->bf16) a.e.out_bf16 = (bf16*)m->h16;
    else { a.e.out = m->h; a.e.out_lo = tc_h ? m->h_lo : nullptr; }
    if ((rc = linear(m, a, FEED_X_NORM, Ly.w_hi[2], Ly.w_lo[2])) != L3_OK) return rc;
    // x = x + h @ Wdown^T                                         llama3.py:102, 259
    a = LinearArgs{};
    a.W = Ly.w2; a.x = m->h; a.rows = ntok; a.N = D; a.K = m->FD; a.src_mul = 1;
    a.epi = EPI_RESID; a.e = base; a.e.out = m->x; a.e.resid = m->x; a.e.ld_out = D;
    if ((rc = tp_row_parallel(m, a, FEED_H, Ly.w_hi[3], Ly.w_lo[3], ntok, tc_rows)) != L3_OK) return rc;
  }
  if (want_logits || want_argmax) {
    // logits = norm(x)[:, -1] @ lm_head^T                         llama3.py:304-307
    LinearArgs a{};
    a.W = m->lm_head; a.x = m->x; a.rows = B; a.N = m->VS; a.K = D;
    a.norm_w = m->norm_final; a.eps = m->cfg.norm_eps; a.src_mul = L; a.src_add = L - 1;
    if (rg && rg->last_rows) a.src_rows = rg->last_rows;  // ragged prefill: each prompt's own last token
    float* lg = m->G > 1 ? m->logits_loc : m->logits;  // under TP: this rank's vocabulary slice
    a.epi = EPI_STORE; a.e = base; a.e.out = lg; a.e.ld_out = m->VS;
    // generate only needs the argmax: the tensor-core LM head then reduces (max, index) in its
    // epilogue and never writes the [B, VS] logits
    const bool fused = want_argmax && !want_logits && m->tc_ok && !linear_rows_supported(B, D);
    if (fused) { a.epi = EPI_ARGMAX; a.e.out = nullptr; a.e.best = m->d_best; a.e.col_offset = m->cfg.tp_rank * m->VS; }
    if ((rc = linear(m, a, FEED_LAST_NORM, m->lm_hi, m->lm_lo)) != L3_OK) return rc;
    if (m->G > 1) {
      // vocabulary-sharded head: ranks merge packed (value, first index) keys with one u64 max
      if (want_argmax) {
        if (!fused) LAUNCH(m, launch_argmax_keys(lg, B, m->VS, m->cfg.tp_rank * m->VS, m->d_best, m->stream));
        if ((rc = tp_allreduce_max_u64(m, m->d_best, B)) != L3_OK) return rc;
        LAUNCH(m, launch_argmax_finalize(m->d_best, B, os.next, os.out64, os.stride, os.step_ptr, m->stream));
      }
      if (want_logits) {
        if ((rc = tp_allgather(m, lg, m->logits_all, (int64_t)B * m->VS)) != L3_OK) return rc;
        LAUNCH(m, launch_gather_permute(m->logits_all, m->G, B, m->VS, m->logits, m->stream));
      }
    } else if (fused)
      LAUNCH(m, launch_argmax_finalize(m->d_best, B, os.next, os.out64, os.stride, os.step_ptr, m->stream));
    else if (want_argmax)  // llama3.py:320
      LAUNCH(m, launch_argmax(m->logits, B, m->VS, os.next, os.out64, os.stride, os.step_ptr, m->stream));
  }
  return L3_OK;
}

// Prefill of [B, L] at start_pos, in chunks of at most cap_tok rows.
static int enqueue_prefill(L3Model* m, const int32_t* d_ids, int B, int L, int start_pos, bool want_logits,
                           bool want_argmax, OutSpec os, const int32_t* d_rows = nullptr, int n_rows = 0,
                           float* d_resid = nullptr) {
  int* d_pos = m->d_scal + 0;
  if (m->ll) {  // a call at position 0 starts its slots afresh; any other must continue them
    const int rc = ll_begin_call(m, B, L, start_pos);
    if (rc != L3_OK) return rc;
  }
  LAUNCH(m, launch_set_int(d_pos, start_pos, m->stream));
  if (d_rows || d_resid)  // chosen rows / the residual trace index the whole block: one chunk (checked by the caller)
    return enqueue_chunk(m, d_ids, L, 0, B, L, want_logits, want_argmax, os, nullptr, d_rows, n_rows, d_resid);
  const int lc_max = std::max(1, m->cap_tok / B);
  for (int l0 = 0; l0 < L; l0 += lc_max) {
    const int lc = std::min(lc_max, L - l0);
    const bool last = l0 + lc >= L;
    int rc = enqueue_chunk(m, d_ids, L, l0, B, lc, last && want_logits, last && want_argmax, os);
    if (rc != L3_OK) return rc;
    if (!last) LAUNCH(m, launch_add_int(d_pos, lc, m->stream));
  }
  return L3_OK;
}

static int check_call(L3Model* m, int B, int L, int start_pos) {
  if (!m) return L3_EINVAL;
  if (!m->finalized) { set_err(m, "model not finalized"); return L3_ESTATE; }
  if (m->G > 1 && !m->comm) { set_err(m, "tensor parallel model: call l3_tp_init first"); return L3_ESTATE; }
  REQUIRE(m, B >= 1 && B <= m->maxB, "batch %d exceeds max_batch_size %d", B, m->maxB);
  REQUIRE(m, L >= 1 && start_pos >= 0 && start_pos + L <= m->M, "start_pos %d + L %d exceeds max_seq_len %d",
          start_pos, L, m->M);
  return L3_OK;
}

extern "C" int l3_forward_dev(L3Model* m, const int32_t* d_ids, int B, int L, int start_pos, float* d_logits_out,
                              int64_t* d_argmax_out) {
  int rc = check_call(m, B, L, start_pos);
  if (rc != L3_OK) return rc;
  CK(m, cudaSetDevice(m->cfg.device));
  if ((rc = enqueue_prefill(m, d_ids, B, L, start_pos, true, d_argmax_out != nullptr,
                            OutSpec{m->d_fwd_arg, 1, m->d_scal + 3, m->d_fwd_next})) != L3_OK) return rc;
  if (d_logits_out)
    CK(m, cudaMemcpyAsync(d_logits_out, m->logits, (size_t)B * m->cfg.vocab_size * 4, cudaMemcpyDeviceToDevice, m->stream));
  if (d_argmax_out)
    CK(m, cudaMemcpyAsync(d_argmax_out, m->d_fwd_arg, (size_t)B * 8, cudaMemcpyDeviceToDevice, m->stream));
  return L3_OK;
}

extern "C" int l3_forward(L3Model* m, const int32_t* ids, int B, int L, int start_pos, float* logits_out,
                          int64_t* argmax_out) {
  int rc = check_call(m, B, L, start_pos);
  if (rc != L3_OK) return rc;
  CK(m, cudaSetDevice(m->cfg.device));
  for (int i = 0; i < B * L; ++i)
    REQUIRE(m, ids[i] >= 0 && ids[i] < m->cfg.vocab_size, "token id %d out of range at %d", ids[i], i);
  // d_fwd_ids, not d_ids: a prompt handed to l3_generate_begin waits in d_ids until the first l3_generate_next
  CK(m, cudaMemcpyAsync(m->d_fwd_ids, ids, (size_t)B * L * 4, cudaMemcpyHostToDevice, m->stream));
  if ((rc = enqueue_prefill(m, m->d_fwd_ids, B, L, start_pos, true, argmax_out != nullptr,
                            OutSpec{m->d_fwd_arg, 1, m->d_scal + 3, m->d_fwd_next})) != L3_OK) return rc;
  if (logits_out)
    CK(m, cudaMemcpyAsync(logits_out, m->logits, (size_t)B * m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->stream));
  if (argmax_out)
    CK(m, cudaMemcpyAsync(argmax_out, m->d_fwd_arg, (size_t)B * 8, cudaMemcpyDeviceToHost, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

extern "C" int l3_forward_rows(L3Model* m, const int32_t* ids, int B, int L, int start_pos, const int32_t* rows, int n_rows,
                               float* logits_out, float* resid_out) {
  int rc = check_call(m, B, L, start_pos);
  if (rc != L3_OK) return rc;
  REQUIRE(m, m->ll != nullptr, "l3_forward_rows needs a handle made by l3_create_stack");
  REQUIRE(m, n_rows >= 0 && (n_rows == 0 || (rows && logits_out)), "rows / logits_out missing");
  REQUIRE(m, (int64_t)B * L <= m->cap_tok, "%d x %d tokens exceed one chunk of %d rows: feed the block in pieces", B, L, m->cap_tok);
  CK(m, cudaSetDevice(m->cfg.device));
  for (int i = 0; i < B * L; ++i)
    REQUIRE(m, ids[i] >= 0 && ids[i] < m->cfg.vocab_size, "token id %d out of range at %d", ids[i], i);
  for (int i = 0; i < n_rows; ++i) REQUIRE(m, rows[i] >= 0 && rows[i] < B * L, "row %d out of range", rows[i]);
  if ((rc = ll_ensure_head_rows(m, n_rows)) != L3_OK) return rc;
  int32_t* d_rows = nullptr;
  float* d_resid = nullptr;
  if (n_rows) {
    CK(m, cudaMalloc((void**)&d_rows, (size_t)n_rows * 4));
    CK(m, cudaMemcpyAsync(d_rows, rows, (size_t)n_rows * 4, cudaMemcpyHostToDevice, m->stream));
  }
  const size_t nres = m->ll->runs.size() * (size_t)B * L * m->D;
  if (resid_out) CK(m, cudaMalloc((void**)&d_resid, nres * 4));
  CK(m, cudaMemcpyAsync(m->d_fwd_ids, ids, (size_t)B * L * 4, cudaMemcpyHostToDevice, m->stream));
  rc = enqueue_prefill(m, m->d_fwd_ids, B, L, start_pos, n_rows > 0, false, OutSpec{m->d_fwd_arg, 1, m->d_scal + 3, m->d_fwd_next},
                       d_rows ? d_rows : nullptr, n_rows, d_resid);
  cudaError_t e = cudaSuccess;
  if (rc == L3_OK && n_rows)
    e = cudaMemcpyAsync(logits_out, m->logits, (size_t)n_rows * m->cfg.vocab_size * 4, cudaMemcpyDeviceToHost, m->stream);
  if (rc == L3_OK && e == cudaSuccess && resid_out) e = cudaMemcpyAsync(resid_out, d_resid, nres * 4, cudaMemcpyDeviceToHost, m->stream);
  const cudaError_t e2 = cudaStreamSynchronize(m->stream);
  if (d_rows) cudaFree(d_rows);
  if (d_resid) cudaFree(d_resid);
  if (rc != L3_OK) return rc;
  CK(m, e);
  CK(m, e2);
  return L3_OK;
}

// ------------------------------------------------------------------------------ greedy loop
// Decode step i >= 1 of Llama.generate: inputs = previous argmax, pos = L + i (llama3.py:316-318).
// All step state lives on the device (d_scal: [0] pos, [1] step, [2] prompt length), so the
// step is one CUDA graph replayed without host involvement.
__global__ void advance_step_kernel(int* scal) {
  pdl_launch();
  pdl_wait();
  const int s = scal[1] + 1;
  scal[1] = s;
  scal[0] = scal[2] + s;
}

// Batch-1 decode: the whole step is one persistent kernel (decode_mega.cu).
static int enqueue_decode_mega(L3Model* m) {
  MegaArgs a{};
  a.layers = (const MegaLayer*)m->d_mega_layers;
  a.NL = m->cfg.n_layers; a.D = m->D; a.HN = m->HN; a.KVHN = m->KVHN; a.HD = m->HD; a.FD = m->FD; a.VS = m->VS; a.M = m->M;
  a.embed = m->embed; a.lm_head = m->lm_head; a.norm_final = m->norm_final; a.eps = m->cfg.norm_eps;
  a.cos_tab = m->cos_tab; a.sin_tab = m->sin_tab;
  a.x = m->x; a.q = m->q; a.ctx = m->ctx; a.h = m->h;
  a.part_o = m->part_o; a.part_ml = m->part_ml; a.attn_cnt = m->attn_cnt;
  a.nsplit = std::max(1, std::min(m->max_split, m->n_sm / m->KVHN));
  a.scal = m->d_scal; a.d_next = m->d_next; a.d_tokens = m->d_tokens; a.d_best = m->d_best;
  a.bar_cnt = m->d_mega_bar; a.bar_gen = m->d_mega_bar + 1;
  a.dbg = m->d_mega_dbg;
  a.tp_rank = m->cfg.tp_rank; a.tp_world = m->G;
  a.ll_words = L3_LL_WORDS;
  a.ll_ctx = m->d_mega_ll + (size_t)2 * L3_LL_WORDS;
  a.ll_xsum = a.ll_ctx + (size_t)m->HN * m->HD;
  if (m->G > 1) {
    L3Comm* c = m->comm;
    for (int p = 0; p < c->world; ++p)
      a.peer_ll[p] = (unsigned long long*)((char*)c->peer_base[p] + tp_ll_off());
    a.epoch = (unsigned*)((char*)c->area + tp_epoch_off()) + 1;
  } else {
    a.peer_ll[0] = m->d_mega_ll;
    a.epoch = m->d_mega_bar + 2;
  }
  LAUNCH(m, launch_decode_mega(a, m->bf16, m->n_sm, m->stream));
  return L3_OK;
}

// Batched decode of a small fp32 model: every layer of the step in ONE cluster-resident kernel (decode_stack.cu:
// the activations of a block of sequences never leave their cluster), then the tensor-core LM head with the
// argmax fused into its epilogue, then next ids / token table / step scalars.  Three launches per step.
static int enqueue_decode_stack(L3Model* m, int B, int part = 0) {
  StackArgs a{};
  a.layers = (const StackLayer*)m->d_stack_layers;
  a.NL = m->cfg.n_layers; a.B = B; a.M = m->M;
  a.embed = (const float*)m->embed; a.norm_final = m->norm_final; a.eps = m->cfg.norm_eps;
  a.cos_tab = m->cos_tab; a.sin_tab = m->sin_tab;
  a.scal = m->d_scal; a.d_next = m->d_next;
  a.xlast_hi = m->xlast; a.xlast_lo = m->xlast_lo;
  a.dbg = m->d_stack_dbg;
  a.dbg_x = m->d_stack_dbgx;
  // measured on the headline (profiles/r02_stack_sweep.jsonl): 64 rows + evict-first 841 k tok/s, both off 822 k, 256 rows 810 k
  static const int pf_rows = [] { const char* v = getenv("L3_STACK_PF"); return v ? atoi(v) : 64; }();
  static const int kv_ef = [] { const char* v = getenv("L3_STACK_KV_EVICT_FIRST"); return v ? atoi(v) : 1; }();
  a.pf_rows = pf_rows; a.kv_evict_first = kv_ef;
  if (part != 2) LAUNCH(m, launch_decode_stack(a, m->D, m->HN, m->HD, m->FD, m->stream));
  if (part == 1) return L3_OK;
  TcGemmArgs t{};
  t.kind = m->D <= 512 ? TC_TF32X3_2 : TC_TF32X3;
  t.A[0] = m->xlast; t.A[1] = m->xlast_lo; t.W[0] = m->lm_hi; t.W[1] = m->lm_lo;
  t.rows = B; t.N = m->VS; t.K = m->D; t.bn = 0; t.epi = EPI_ARGMAX;
  t.e.best = m->d_best; t.e.col_offset = 0; t.e.ld_out = m->VS;
  LAUNCH(m, launch_gemm_tc(t, m->stream));
  if (part == 2) return L3_OK;
  LAUNCH(m, launch_stack_finalize(m->d_best, B, m->d_next, m->d_tokens, m->M, m->d_scal, m->stream));
  return L3_OK;
}

static int enqueue_decode_nodes(L3Model* m, int B, int ragged, int eos) {
  if (ragged) {  // per-sequence positions (l3_generate_ragged): never the batch-1 kernel
    LAUNCH(m, launch_ragged_advance(m->d_scal, m->d_rowlen, ragged == 1 ? 0 : -1, B, m->d_rowpos, m->stream));
    Ragged rg{m->d_rowpos, nullptr, nullptr};
    int rc = enqueue_chunk(m, m->d_next, 1, 0, B, 1, false, true, OutSpec{m->d_tokens, m->M, m->d_scal + 1, m->d_next}, &rg);
    if (rc != L3_OK) return rc;
    if (eos >= 0) LAUNCH(m, launch_ragged_eos(m->d_next, m->d_done, eos, B, m->d_tokens, m->M, m->d_scal + 1, m->stream));
    return L3_OK;
  }
  if (m->stack_ok && B >= m->stack_min_B) return enqueue_decode_stack(m, B);
  // under tensor parallelism the kernel runs the peer-memory exchange itself (needs the mapped slots)
  if (B == 1 && m->mega_ok && m->D <= L3_LL_VEC && (m->G == 1 || (m->comm && m->comm->oneshot)))
    return enqueue_decode_mega(m);
  LAUNCH(m, launch_k(advance_step_kernel, dim3(1), dim3(1), 0, m->stream, m->d_scal));
  return enqueue_chunk(m, m->d_next, 1, 0, B, 1, false, true, OutSpec{m->d_tokens, m->M, m->d_scal + 1, m->d_next});
}

static int decode_step(L3Model* m, int B, int ragged = 0, int eos = -1) {
  if (m->ll)
    for (int b = 0; b < B; ++b) m->ll->slot_pos[b] += 1;
  L3Graph* g = nullptr;
  const int key = ragged ? ragged + 4 * (eos + 1) : 0;  // the EOS id is baked into the captured node
  for (auto& it : m->graphs)
    if (it.B == B && it.ragged == key) g = &it;
  if (!g) { m->graphs.push_back(L3Graph{B}); g = &m->graphs.back(); g->ragged = key; }
  if (m->cfg.flags & L3_FLAG_NO_GRAPH) return enqueue_decode_nodes(m, B, ragged, eos);
  if (g->exec) {
    CK(m, cudaGraphLaunch(g->exec, m->stream));
    m->launch_acc += g->nodes;
    return L3_OK;
  }
  if (!g->warmed) {  // first step runs eagerly (sets function attributes, validates the launches)
    g->warmed = true;
    return enqueue_decode_nodes(m, B, ragged, eos);
  }
  const int64_t before = m->launch_acc;
  CK(m, cudaStreamBeginCapture(m->stream, cudaStreamCaptureModeThreadLocal));
  int rc = enqueue_decode_nodes(m, B, ragged, eos);
  cudaError_t e = cudaStreamEndCapture(m->stream, &g->graph);
  if (rc != L3_OK) return rc;
  CK(m, e);
  g->nodes = m->launch_acc - before;
  m->launch_acc = before;
  CK(m, cudaGraphInstantiate(&g->exec, g->graph, 0));
  CK(m, cudaGraphLaunch(g->exec, m->stream));
  m->launch_acc += g->nodes;
  return L3_OK;
}

static int generate_begin_dev(L3Model* m, const int32_t* d_ids, int B, int L) {
  // d_scal[2] = position base of the decode steps: step i runs at pos = base + i.  base = L is the
  // reference generator's schedule (llama3.py:316-318, slot L skipped); base = L - 1 is the
  // functional implementation's (llama3_simple.py:279).
  int h[4] = {0, 0, L + m->gen_off, 0};
  CK(m, cudaMemcpyAsync(m->d_scal, h, sizeof h, cudaMemcpyHostToDevice, m->stream));
  m->gen_B = B;
  m->gen_L = L;
  m->gen_step = 0;
  return enqueue_prefill(m, d_ids, B, L, 0, false, true, OutSpec{m->d_tokens, m->M, m->d_scal + 1, m->d_next});
}

extern "C" int l3_generate_greedy_dev(L3Model* m, const int32_t* d_ids, int B, int L, int max_new_tokens,
                                      int64_t* d_out) {
  int rc = check_call(m, B, L, 0);
  if (rc != L3_OK) return rc;
  REQUIRE(m, max_new_tokens <= m->M, "max_new_tokens %d exceeds max_seq_len %d", max_new_tokens, m->M);
  const int n_out = max_new_tokens - L;
  if (n_out <= 0) return L3_OK;
  CK(m, cudaSetDevice(m->cfg.device));
  m->gen_off = m->ll ? -1 : 0;  // layer-list decoders generate at contiguous positions
  if ((rc = generate_begin_dev(m, d_ids, B, L)) != L3_OK) return rc;
  for (int i = 1; i < n_out; ++i)
    if ((rc = decode_step(m, B)) != L3_OK) return rc;
  CK(m, cudaMemcpy2DAsync(d_out, (size_t)n_out * 8, m->d_tokens, (size_t)m->M * 8, (size_t)n_out * 8, B,
                          cudaMemcpyDeviceToDevice, m->stream));
  return L3_OK;
}

extern "C" int l3_generate_greedy(L3Model* m, const int32_t* ids, int B, int L, int max_new_tokens, int64_t* out) {
  int rc = check_call(m, B, L, 0);
  if (rc != L3_OK) return rc;
  REQUIRE(m, max_new_tokens <= m->M, "max_new_tokens %d exceeds max_seq_len %d", max_new_tokens, m->M);
  const int n_out = max_new_tokens - L;
  if (n_out <= 0) return L3_OK;
  CK(m, cudaSetDevice(m->cfg.device));
  for (int i = 0; i < B * L; ++i)
    REQUIRE(m, ids[i] >= 0 && ids[i] < m->cfg.vocab_size, "token id %d out of range at %d", ids[i], i);
  CK(m, cudaMemcpyAsync(m->d_ids, ids, (size_t)B * L * 4, cudaMemcpyHostToDevice, m->stream));
  m->gen_off = m->ll ? -1 : 0;  // layer-list decoders generate at contiguous positions
  if ((rc = generate_begin_dev(m, m->d_ids, B, L)) != L3_OK) return rc;
  for (int i = 1; i < n_out; ++i)
    if ((rc = decode_step(m, B)) != L3_OK) return rc;
  CK(m, cudaMemcpy2DAsync(out, (size_t)n_out * 8, m->d_tokens, (size_t)m->M * 8, (size_t)n_out * 8, B,
                          cudaMemcpyDeviceToHost, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}

// Greedy generation for prompts of DIFFERENT lengths (the reference handles equal
// lengths only and checks EOS for row 0 in the caller, llama3.py:341-343).  Each sequence behaves exactly
// as if it ran alone through Llama.generate (pos_offset 0) or llama_generate (pos_offset -1): the
// right-padded prompt rows are prefilled together, padding leaves the KV cache untouched, the LM head
// reads every prompt's own last token, and decode step i of sequence b runs at pos = len[b] + off + i.
extern "C" int l3_generate_ragged(L3Model* m, const int32_t* ids, const int32_t* lens, int B, int Lmax, int max_new_tokens,
                                  int pos_offset, int eos_id, int64_t* out) {
  int rc = check_call(m, B, Lmax, 0);
  if (rc != L3_OK) return rc;
  REQUIRE(m, pos_offset == 0 || pos_offset == -1, "pos_offset must be 0 (llama3.py) or -1 (llama3_simple.py)");
  REQUIRE(m, !m->ll, "ragged batches are not built for layer-list handles");
  REQUIRE(m, B <= 1024, "at most 1024 sequences per ragged batch");
  REQUIRE(m, (int64_t)B * Lmax <= m->cap_tok, "ragged prompts must fit one chunk: %d x %d > %d rows", B, Lmax, m->cap_tok);
  REQUIRE(m, max_new_tokens >= 1, "max_new_tokens must be >= 1");
  int lmax = 0;
  for (int b = 0; b < B; ++b) {
    REQUIRE(m, lens[b] >= 1 && lens[b] <= Lmax, "prompt %d has length %d outside [1, %d]", b, lens[b], Lmax);
    lmax = std::max(lmax, (int)lens[b]);
    for (int t = 0; t < lens[b]; ++t)
      REQUIRE(m, ids[b * Lmax + t] >= 0 && ids[b * Lmax + t] < m->cfg.vocab_size, "token id out of range in prompt %d", b);
  }
  REQUIRE(m, lmax + pos_offset + max_new_tokens <= m->M, "longest prompt %d + %d new tokens exceed max_seq_len %d", lmax,
          max_new_tokens, m->M);
  REQUIRE(m, eos_id < m->cfg.vocab_size, "eos_id out of range");
  CK(m, cudaSetDevice(m->cfg.device));
  std::vector<int32_t> padded((size_t)B * Lmax);
  for (int b = 0; b < B; ++b)
    for (int t = 0; t < Lmax; ++t) padded[(size_t)b * Lmax + t] = t < lens[b] ? ids[b * Lmax + t] : 0;
  CK(m, cudaMemcpyAsync(m->d_ids, padded.data(), padded.size() * 4, cudaMemcpyHostToDevice, m->stream));
  CK(m, cudaMemcpyAsync(m->d_rowlen, lens, (size_t)B * 4, cudaMemcpyHostToDevice, m->stream));
  int h[4] = {0, 0, 0, 0};
  CK(m, cudaMemcpyAsync(m->d_scal, h, sizeof h, cudaMemcpyHostToDevice, m->stream));
  LAUNCH(m, launch_ragged_setup(m->d_rowlen, B, Lmax, m->d_lastrow, m->d_done, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));  // `padded` leaves scope
  Ragged rg{nullptr, m->d_rowlen, m->d_lastrow};
  if ((rc = enqueue_chunk(m, m->d_ids, Lmax, 0, B, Lmax, false, true, OutSpec{m->d_tokens, m->M, m->d_scal + 1, m->d_next}, &rg)) != L3_OK)
    return rc;
  const int eos = eos_id < 0 ? -1 : eos_id;
  if (eos >= 0) LAUNCH(m, launch_ragged_eos(m->d_next, m->d_done, eos, B, m->d_tokens, m->M, m->d_scal + 1, m->stream));
  for (int i = 1; i < max_new_tokens; ++i)
    if ((rc = decode_step(m, B, pos_offset == 0 ? 1 : 2, eos)) != L3_OK) return rc;
  CK(m, cudaMemcpy2DAsync(out, (size_t)max_new_tokens * 8, m->d_tokens, (size_t)m->M * 8, (size_t)max_new_tokens * 8, B,
                          cudaMemcpyDeviceToHost, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  m->gen_B = 0;
  return L3_OK;
}

extern "C" int l3_generate_begin(L3Model* m, const int32_t* ids, int B, int L) { return l3_generate_begin_ex(m, ids, B, L, 0); }

extern "C" int l3_generate_begin_ex(L3Model* m, const int32_t* ids, int B, int L, int pos_offset) {
  int rc = check_call(m, B, L, 0);
  if (rc != L3_OK) return rc;
  REQUIRE(m, pos_offset == 0 || pos_offset == -1, "pos_offset must be 0 (llama3.py) or -1 (llama3_simple.py)");
  m->pend_off = m->ll ? -1 : pos_offset;
  CK(m, cudaSetDevice(m->cfg.device));
  for (int i = 0; i < B * L; ++i)
    REQUIRE(m, ids[i] >= 0 && ids[i] < m->cfg.vocab_size, "token id %d out of range at %d", ids[i], i);
  m->gen_B = 0;  // the prefill itself is enqueued by the first l3_generate_next (lazy, like the generator)
  CK(m, cudaMemcpyAsync(m->d_ids, ids, (size_t)B * L * 4, cudaMemcpyHostToDevice, m->stream));
  m->pend_B = B;
  m->pend_L = L;
  return L3_OK;
}

extern "C" int l3_generate_next(L3Model* m, int64_t* out_B) {
  if (!m || !m->finalized) return L3_ESTATE;
  CK(m, cudaSetDevice(m->cfg.device));
  int rc;
  if (m->pend_B) {
    const int B = m->pend_B, L = m->pend_L;
    m->pend_B = 0;
    m->gen_off = m->pend_off;
    if ((rc = generate_begin_dev(m, m->d_ids, B, L)) != L3_OK) return rc;
  } else {
    if (!m->gen_B) { set_err(m, "l3_generate_next without l3_generate_begin"); return L3_ESTATE; }
    m->gen_step += 1;
    REQUIRE(m, m->gen_L + m->gen_off + m->gen_step < m->M, "position %d reaches max_seq_len %d",
            m->gen_L + m->gen_off + m->gen_step, m->M);
    if ((rc = decode_step(m, m->gen_B)) != L3_OK) return rc;
  }
  CK(m, cudaMemcpyAsync(m->h_next, m->d_next, (size_t)m->gen_B * 4, cudaMemcpyDeviceToHost, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  for (int b = 0; b < m->gen_B; ++b) out_B[b] = m->h_next[b];
  return L3_OK;
}

// ------------------------------------------------------------------------------ measurement helpers
extern "C" int l3_sync(L3Model* m) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}
extern "C" int l3_timer_start(L3Model* m) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaStreamSynchronize(m->stream));
  CK(m, cudaEventRecord(m->ev0, m->stream));
  return L3_OK;
}
extern "C" int l3_timer_stop(L3Model* m, float* ms_out) {
  if (!m) return L3_EINVAL;
  CK(m, cudaEventRecord(m->ev1, m->stream));
  CK(m, cudaEventSynchronize(m->ev1));
  CK(m, cudaEventElapsedTime(ms_out, m->ev0, m->ev1));
  return L3_OK;
}
extern "C" int l3_dev_alloc(L3Model* m, int64_t bytes, void** out) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaMalloc(out, (size_t)bytes));
  return L3_OK;
}
extern "C" int l3_dev_free(L3Model* m, void* p) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaFree(p));
  return L3_OK;
}
extern "C" int l3_memcpy_h2d(L3Model* m, void* dst, const void* src, int64_t bytes) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyHostToDevice, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}
extern "C" int l3_memcpy_d2h(L3Model* m, void* dst, const void* src, int64_t bytes) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaMemcpyAsync(dst, src, (size_t)bytes, cudaMemcpyDeviceToHost, m->stream));
  CK(m, cudaStreamSynchronize(m->stream));
  return L3_OK;
}
extern "C" int l3_flush_l2(L3Model* m) {
  if (!m) return L3_EINVAL;
  CK(m, cudaSetDevice(m->cfg.device));
  const size_t bytes = (size_t)256 << 20;  // 2x the 126 MB L2
  if (!m->l2buf) CK(m, cudaMalloc(&m->l2buf, bytes));
  m->l2_phase ^= 1;
  CK(m, cudaMemsetAsync(m->l2buf, m->l2_phase, bytes, m->stream));
  return L3_OK;
}
extern "C" int l3_debug_mega_timeline(L3Model* m, uint64_t* out, int64_t capacity) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, m->d_mega_dbg != nullptr, "timeline off: set L3_MEGA_DBG=1 before creating the model");
  REQUIRE(m, capacity >= (int64_t)m->n_sm * 512, "need room for %d x 512 stamps", m->n_sm);
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaStreamSynchronize(m->stream));
  CK(m, cudaMemcpy(out, m->d_mega_dbg, (size_t)m->n_sm * 512 * 8, cudaMemcpyDeviceToHost));
  return L3_OK;
}

extern "C" int l3_debug_stack(L3Model* m, int which, void* out, int64_t capacity_bytes) {
  if (!m) return L3_EINVAL;
  REQUIRE(m, m->d_stack_dbg != nullptr, "stack debug off: set L3_STACK_DBG=1 before creating the model");
  const int spc = decode_stack_seqs_per_cluster();
  const size_t bytes = which == 0 ? (size_t)((m->maxB + spc - 1) / spc) * 8 * 128 * 8 : (size_t)m->cfg.n_layers * 4 * m->maxB * m->D * 4;
  REQUIRE(m, capacity_bytes >= (int64_t)bytes, "need %zu bytes", bytes);
  CK(m, cudaSetDevice(m->cfg.device));
  CK(m, cudaStreamSynchronize(m->stream));
  CK(m, cudaMemcpy(out, which == 0 ? (void*)m->d_stack_dbg : (void*)m->d_stack_dbgx, bytes, cudaMemcpyDeviceToHost));
  return L3_OK;
}

extern "C" int l3_launch_count(L3Model* m, int64_t* out, int reset) {
  if (!m) return L3_EINVAL;
  *out = m->launch_acc;
  if (reset) m->launch_acc = 0;
  return L3_OK;
}

extern "C" int l3_bench_kernel(L3Model* m, int which, int B, int pos, int iters, float* avg_ms) {
  int rc = check_call(m, B, 1, pos);
  if (rc != L3_OK) return rc;
  REQUIRE(m, !m->ll, "l3_bench_kernel times kernels of the Llama path");
  CK(m, cudaSetDevice(m->cfg.device));
  REQUIRE(m, iters >= 1, "iters must be >= 1");
  int* d_pos = m->d_scal + 0;
  CK(m, launch_set_int(d_pos, pos, m->stream));
  EpiArgs base{};
  base.cos_tab = m->cos_tab; base.sin_tab = m->sin_tab; base.pos_ptr = d_pos;
  base.L = 1; base.HD = m->HD; base.HN = m->HN; base.KVHN = m->KVHN; base.M = m->M;
  auto once = [&](int it) -> int {
    if (which == 0) {  // decode attention, rotating over layers so that the KV set exceeds L2
      auto& Ly = m->layers[it % m->layers.size()];
      AttnArgs at{};
      at.q = m->q; at.cache_k = Ly.ck; at.cache_v = Ly.cv; at.out = m->ctx; at.pos_ptr = d_pos;
      at.B = B; at.L = 1; at.HN = m->HN; at.KVHN = m->KVHN; at.HD = m->HD; at.M = m->M;
      at.part_o = m->part_o; at.part_ml = m->part_ml; at.nsplit = pick_nsplit(m, B); at.counters = m->attn_cnt;
      CK(m, launch_attn_decode(at, m->bf16, m->stream));
    } else if (which == 1) {  // LM head on B rows
      LinearArgs a{};
      a.W = m->lm_head; a.x = m->x; a.rows = B; a.N = m->VS; a.K = m->D;
      a.norm_w = m->norm_final; a.eps = m->cfg.norm_eps; a.src_mul = 1; a.src_add = 0;
      a.epi = EPI_STORE; a.e = base; a.e.out = m->logits; a.e.ld_out = m->VS;
      const int64_t keep = m->launch_acc;
      int r = linear(m, a, FEED_LAST_NORM, m->lm_hi, m->lm_lo);
      m->launch_acc = keep;
      return r;
    } else if (which == 3) {  // the two residual projections of a layer (Wo, Wdown): ONE kernel symbol, 2 launches
      auto& Ly = m->layers[it % m->layers.size()];
      const int64_t keep = m->launch_acc;
      LinearArgs a{};
      a.W = Ly.wo; a.x = m->ctx; a.rows = B; a.N = m->D; a.K = m->HN * m->HD; a.src_mul = 1;
      a.epi = EPI_RESID; a.e = base; a.e.out = m->q; a.e.resid = m->x; a.e.ld_out = m->D;  // q as a scratch output
      int r = linear(m, a, FEED_CTX, Ly.w_hi[1], Ly.w_lo[1]);
      if (r != L3_OK) return r;
      a = LinearArgs{};
      a.W = Ly.w2; a.x = m->h; a.rows = B; a.N = m->D; a.K = m->FD; a.src_mul = 1;
      a.epi = EPI_RESID; a.e = base; a.e.out = m->q; a.e.resid = m->x; a.e.ld_out = m->D;
      r = linear(m, a, FEED_H, Ly.w_hi[3], Ly.w_lo[3]);
      m->launch_acc = keep;
      return r;
    } else {  // FFN gate/up + down of layer (it % n_layers)
      auto& Ly = m->layers[it % m->layers.size()];
      LinearArgs a{};
      a.W = Ly.w13; a.x = m->x; a.rows = B; a.N = 2 * m->FD; a.K = m->D;
      a.norm_w = Ly.norm_post; a.eps = m->cfg.norm_eps; a.src_mul = 1;
      a.epi = EPI_SWIGLU; a.e = base; a.e.ld_out = m->FD;
      const bool tc_h = m->tc_ok && !linear_rows_supported(B, m->FD);
      if (tc_h && m->bf16) a.e.out_bf16 = (bf16*)m->h16;
      else { a.e.out = m->h; a.e.out_lo = tc_h ? m->h_lo : nullptr; }
      const int64_t keep = m->launch_acc;
      int r = linear(m, a, FEED_X_NORM, Ly.w_hi[2], Ly.w_lo[2]);
      if (r != L3_OK) return r;
      a = LinearArgs{};
      a.W = Ly.w2; a.x = m->h; a.rows = B; a.N = m->D; a.K = m->FD; a.src_mul = 1;
      a.epi = EPI_STORE; a.e = base; a.e.out = m->q; a.e.ld_out = m->D;
      r = linear(m, a, FEED_H, Ly.w_hi[3], Ly.w_lo[3]);
      m->launch_acc = keep;
      return r;
    }
    return L3_OK;
  };
  if (which == 4 || which == 5) {
    // The batched decode path's two kernels, each timed ALONE with the L2 flushed before every launch:
    // 4 = decode_stack_kernel (every layer of one decode step at position `pos`), 5 = its LM head (256-wide tiles,
    // fused argmax).  The step scalars and token ids are set so that the kernel sees a valid state; the K / V row it
    // appends lands at `pos`.
    REQUIRE(m, m->stack_ok && B >= m->stack_min_B, "the cluster-resident decode path is not active for this model / batch");
    REQUIRE(m, pos >= 1, "pos must be >= 1");
    int hs[4] = {pos, 0, pos - 1, 0};
    CK(m, cudaMemcpyAsync(m->d_scal, hs, sizeof hs, cudaMemcpyHostToDevice, m->stream));
    CK(m, cudaMemsetAsync(m->d_next, 0, (size_t)B * 4, m->stream));
    CK(m, cudaStreamSynchronize(m->stream));
    float total = 0.f;
    const int64_t keep = m->launch_acc;
    for (int i = 0; i < iters + 2; ++i) {
      if ((rc = l3_flush_l2(m)) != L3_OK) return rc;
      if (which == 5 && (rc = enqueue_decode_stack(m, B, 1)) != L3_OK) return rc;  // produces the LM head's operands
      CK(m, cudaEventRecord(m->ev0, m->stream));
      if ((rc = enqueue_decode_stack(m, B, which == 4 ? 1 : 2)) != L3_OK) return rc;
      CK(m, cudaEventRecord(m->ev1, m->stream));
      CK(m, cudaEventSynchronize(m->ev1));
      float ms = 0.f;
      CK(m, cudaEventElapsedTime(&ms, m->ev0, m->ev1));
      if (i >= 2) total += ms;
      CK(m, cudaMemsetAsync(m->d_best, 0, (size_t)B * 8, m->stream));
    }
    m->launch_acc = keep;
    *avg_ms = total / iters;
    return L3_OK;
  }
  for (int i = 0; i < 3; ++i)
    if ((rc = once(i)) != L3_OK) return rc;
  CK(m, cudaStreamSynchronize(m->stream));
  CK(m, cudaEventRecord(m->ev0, m->stream));
  for (int i = 0; i < iters; ++i)
    if ((rc = once(i)) != L3_OK) return rc;
  CK(m, cudaEventRecord(m->ev1, m->stream));
  CK(m, cudaEventSynchronize(m->ev1));
  float ms = 0.f;
  CK(m, cudaEventElapsedTime(&ms, m->ev0, m->ev1));
  *avg_ms = ms / iters;
  return L3_OK;
}
