// Native forward of the dense Qwen3 serving stack: one host call issues all the kernels of a layer
// half (or of a whole decode step), so the per-launch cost is a C function call instead of a trip
// through the Python wrappers (~10 us each: an 8B model's 36 layers x ~25 launches made a prefill
// or eager decode step host-bound at 10+ ms).
//
//   bb_serve_begin      embedding -> residual stream
//   bb_serve_pre_attn   (x + delta) -> RMSNorm -> QKV projection -> QK-norm + RoPE -> KV append
//   bb_serve_post_attn  attention output -> Wo -> all-reduce -> (+x) RMSNorm -> gate/up -> SwiGLU
//                       -> down -> all-reduce
//   bb_serve_finish     final RMSNorm of (x + delta)
//   bb_serve_decode     begin + every layer with split-KV paged attention + finish, one call
//
// Between pre_attn and post_attn the caller runs attention (flash kernel over the chunk, or over
// gathered pages) from work->qk / work->qkv into work->o.  Projections are bf16 or W8A8 (per-token
// dynamic activation scales, per-channel weight scales).  With a tensor-parallel group the two
// row-parallel outputs of a layer are summed by the two-shot peer all-reduce; its result buffers
// alternate, and `state->parity` carries which one is next across calls.
// Reference for the step sequence: crates/qwen3/src/serve.rs:1194-1304 (batched decode steps),
// :1557-1623 (chunked prefill).
#include <cmath>
#include <cstdint>

#include "../common/host.hpp"

using namespace bb;

extern "C" {
int bb_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* h_out, float* rstd,
                   int rows, int d, float eps, void* stream);
int bb_quant_rows(const void* x, void* q, float* scale, int rows, int k, int dtype, void* stream);
int bb_gemm_bf16(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
                 int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, float alpha, int bn,
                 int max_ctas, void* stream);
int bb_gemm_i8(const void* A, const void* B, void* C, const float* scale_m, const float* scale_n,
               int M, int N, int K, int lda, int ldb, int ldc, int bn, int max_ctas, void* stream);
int bb_qknorm_rope_fwd(const void* x, int ldx, const void* w_q, const void* w_k, const float* cos_t,
                       const float* sin_t, const int* pos, void* out, int ldo, float* rstd,
                       int n_tok, int hq, int hk, int hd, float eps, void* stream);
int bb_kv_append(const void* k, int ldk, const void* v, int ldv, const int* slots, void* kc,
                 void* vc, int n, int hk, int hd, int bs, void* stream);
int bb_kv_append_i8(const void* k, int ldk, const void* v, int ldv, const int* slots, void* kc,
                    void* vc, float* ks, float* vs, const float* clip, int n, int hk, int hd,
                    int bs, void* stream);
int bb_paged_decode(const void* q, int ldq, const void* kc, const void* vc, const int* block_tables,
                    int max_blocks, const int* seqlens, void* out, int ldo, float* part_o,
                    float* part_ml, int B, int hq, int hk, int hd, int bs, int splits, float scale,
                    void* stream);
int bb_paged_decode_i8(const void* q, int ldq, const void* kc, const void* vc, const float* ks,
                       const float* vs, const int* block_tables, int max_blocks, const int* seqlens,
                       void* out, int ldo, float* part_o, float* part_ml, int B, int hq, int hk,
                       int hd, int bs, int splits, float scale, void* stream);
int bb_swiglu_fwd(const void* gu, void* h, long rows, int ff, void* stream);
int bb_rmsnorm_q8(const void* x, const void* res, const void* w, void* h_out, void* q, float* scale,
                  int rows, int d, float eps, void* stream);
int bb_swiglu_q8(const void* gu, void* q, float* scale, int rows, int ff, void* stream);
int bb_embed_fwd(const int* tok, const void* emb, const void* pos_emb, int T, void* out, long n_tok,
                 int d, int vocab, void* stream);
int bb_tp_allreduce2(const uint64_t* stage_ptrs, const uint64_t* result_ptrs,
                     const uint64_t* sig_ptrs, const void* x, long n, int rank, int world,
                     unsigned int* epoch_dev, unsigned int* counters, double wait_seconds,
                     void* stream);
}

// The structs below are mirrored field for field by ctypes.Structure classes in
// brain_b200/serve/native.py.
struct BbLin {
  const void* w;       // [n, k] bf16, or int8 when scale != null
  const float* scale;  // per-output-channel weight scales (W8A8) or null (bf16)
  const float* bias;   // fp32 [n] or null (bf16 projections only)
  int n, k;
};

struct BbServeLayer {
  const void *ln1, *ln2, *q_norm, *k_norm;   // q_norm / k_norm may be null
  BbLin qkv, wo, gate_up, down;
  void *kc, *vc;             // KV pools of this layer
  float *ks, *vs;            // int8 KV: per-row scales
  const float* kv_clip;      // int8 KV: [2, hk] ceilings or null
};

struct BbServeCfg {
  int d_model, hq, hk, hd, ff, block_size, kv_int8, n_layers;
  float eps;
  int tp_world, tp_rank;
  int fuse_quant;            // W8A8: norms and SwiGLU emit int8 rows + scales directly
  const float *cos_t, *sin_t;
  const BbServeLayer* layers;
  const uint64_t* stage_ptrs;
  const uint64_t* res_ptrs[2];
  const uint64_t* sig_ptrs;
  void* res[2];              // this rank's two all-reduce result buffers
  unsigned int* epoch_dev;
  unsigned int* counters;
  double wait_seconds;
  long ar_cap;               // elements each staging / result buffer holds
};

struct BbServeWork {         // device scratch for `rows` rows
  void *xa, *xb;             // residual stream, ping-pong [rows, d]
  void* h;                   // normed activations [rows, d]
  void* qkv;                 // [rows, (hq + 2 hk) hd]
  void* qk;                  // [rows, (hq + hk) hd]  normed + rotated q | k
  void* o;                   // [rows, hq hd]         attention output
  void* proj;                // [rows, d]
  void* mlp;                 // [rows, d]
  void* gu;                  // [rows, 2 ff]
  void* act;                 // [rows, ff]
  void* xq;                  // int8 [rows, max(d, ff, hq hd)]
  float* sx;                 // [rows]
  float* rstd;               // [rows (hq + hk)]
  float* part_o;             // decode: [rows, hq, splits, hd]
  float* part_ml;            // decode: [rows, hq, splits, 2]
  int rows, splits;
};

struct BbServeState {
  void* x;       // residual stream [n, d]
  void* delta;   // last MLP output not yet added to x (null before the first layer)
  int parity;    // which all-reduce result buffer is next
  int n_allreduce;   // all-reduces issued through this state (the caller keeps its own count in step)
};

namespace {

#define BB_TRY(expr)          \
  do {                        \
    int rc_ = (expr);         \
    if (rc_ != 0) return rc_; \
  } while (0)

int linear(const BbLin& L, const void* x, int ldx, void* y, int rows, const BbServeWork& w, void* stream);

// y = (w.xq * w.sx) . W^T for rows already quantised into the scratch.
int linear_q8(const BbLin& L, void* y, int rows, const BbServeWork& w, void* stream) {
  return bb_gemm_i8(w.xq, L.w, y, w.sx, L.scale, rows, L.n, L.k, L.k, L.k, L.n, 0, 0, stream);
}

// h = RMSNorm(x [+ res]) * g followed by the projection L; with W8A8 and fusion on, the norm emits
// the int8 rows itself (w.h is then not written).
int norm_linear(const BbServeCfg& c, const BbLin& L, const void* x, const void* res, const void* g,
                void* h_out, void* y, int rows, const BbServeWork& w, void* stream) {
  if (c.fuse_quant && L.scale && !L.bias) {
    const int rc = bb_rmsnorm_q8(x, res, g, h_out, w.xq, w.sx, rows, c.d_model, c.eps, stream);
    if (rc == BB_OK) return linear_q8(L, y, rows, w, stream);
    if (rc != BB_ESIZE) return rc;
  }
  BB_TRY(bb_rmsnorm_fwd(x, res, g, w.h, h_out, w.rstd, rows, c.d_model, c.eps, stream));
  return linear(L, w.h, c.d_model, y, rows, w, stream);
}

int linear(const BbLin& L, const void* x, int ldx, void* y, int rows, const BbServeWork& w,
           void* stream) {
  if (L.scale) {
    if (L.bias || ldx != L.k) return BB_EARG;
    BB_TRY(bb_quant_rows(x, w.xq, w.sx, rows, L.k, 0, stream));
    return bb_gemm_i8(w.xq, L.w, y, w.sx, L.scale, rows, L.n, L.k, L.k, L.k, L.n, 0, 0, stream);
  }
  return bb_gemm_bf16(x, L.w, y, L.bias, rows, L.n, L.k, ldx, L.k, L.n, 0, 0, 0, 1.0f, 0, 0, stream);
}

// Sum `x` [n elements] over the tensor-parallel group; returns where the result lives.
int all_reduce(const BbServeCfg& c, BbServeState& s, void* x, long n, void** out, void* stream) {
  if (c.tp_world <= 1) {
    *out = x;
    return BB_OK;
  }
  if (n > c.ar_cap || n % (8L * c.tp_world)) return BB_ESIZE;
  const int which = s.parity & 1;
  BB_TRY(bb_tp_allreduce2(c.stage_ptrs, c.res_ptrs[which], c.sig_ptrs, x, n, c.tp_rank, c.tp_world,
                          c.epoch_dev, c.counters, c.wait_seconds, stream));
  *out = c.res[which];
  s.parity ^= 1;
  s.n_allreduce += 1;
  return BB_OK;
}

int pre_attn(const BbServeCfg& c, int li, const BbServeWork& w, const int* pos, const int* slots,
             int n, BbServeState& s, void* stream) {
  const BbServeLayer& L = c.layers[li];
  const int d = c.d_model, qkv_ld = (c.hq + 2 * c.hk) * c.hd, qk_ld = (c.hq + c.hk) * c.hd;
  if (s.delta) {
    void* xn = (s.x == w.xa) ? w.xb : w.xa;
    BB_TRY(norm_linear(c, L.qkv, s.delta, s.x, L.ln1, xn, w.qkv, n, w, stream));
    s.x = xn;
    s.delta = nullptr;
  } else {
    BB_TRY(norm_linear(c, L.qkv, s.x, nullptr, L.ln1, nullptr, w.qkv, n, w, stream));
  }
  BB_TRY(bb_qknorm_rope_fwd(w.qkv, qkv_ld, L.q_norm, L.k_norm, c.cos_t, c.sin_t, pos, w.qk, qk_ld,
                            L.q_norm ? w.rstd : nullptr, n, c.hq, c.hk, c.hd, c.eps, stream));
  const char* k = static_cast<const char*>(w.qk) + (size_t)c.hq * c.hd * 2;
  const char* v = static_cast<const char*>(w.qkv) + (size_t)qk_ld * 2;
  if (c.kv_int8)
    return bb_kv_append_i8(k, qk_ld, v, qkv_ld, slots, L.kc, L.vc, L.ks, L.vs, L.kv_clip, n, c.hk,
                           c.hd, c.block_size, stream);
  return bb_kv_append(k, qk_ld, v, qkv_ld, slots, L.kc, L.vc, n, c.hk, c.hd, c.block_size, stream);
}

int post_attn(const BbServeCfg& c, int li, const BbServeWork& w, int n, BbServeState& s,
              void* stream) {
  const BbServeLayer& L = c.layers[li];
  const int d = c.d_model;
  void* a = nullptr;
  BB_TRY(linear(L.wo, w.o, c.hq * c.hd, w.proj, n, w, stream));
  BB_TRY(all_reduce(c, s, w.proj, (long)n * d, &a, stream));
  void* xn = (s.x == w.xa) ? w.xb : w.xa;
  BB_TRY(norm_linear(c, L.gate_up, a, s.x, L.ln2, xn, w.gu, n, w, stream));
  s.x = xn;
  int rq = BB_ESIZE;
  if (c.fuse_quant && L.down.scale && !L.down.bias) {
    rq = bb_swiglu_q8(w.gu, w.xq, w.sx, n, c.ff, stream);
    if (rq == BB_OK) BB_TRY(linear_q8(L.down, w.mlp, n, w, stream));
    else if (rq != BB_ESIZE) return rq;
  }
  if (rq != BB_OK) {
    BB_TRY(bb_swiglu_fwd(w.gu, w.act, n, c.ff, stream));
    BB_TRY(linear(L.down, w.act, c.ff, w.mlp, n, w, stream));
  }
  void* m = nullptr;
  BB_TRY(all_reduce(c, s, w.mlp, (long)n * d, &m, stream));
  s.delta = m;
  return BB_OK;
}

}  // namespace

BB_API int bb_serve_begin(const BbServeCfg* c, const BbServeWork* w, const void* tok_emb, int vocab,
                          const int* tokens, int n, BbServeState* s, void* stream) {
  if (!c || !w || !s || n <= 0 || n > w->rows) return BB_EARG;
  BB_TRY(bb_embed_fwd(tokens, tok_emb, nullptr, 1, w->xa, n, c->d_model, vocab, stream));
  s->x = w->xa;
  s->delta = nullptr;
  return BB_OK;
}

BB_API int bb_serve_pre_attn(const BbServeCfg* c, int li, const BbServeWork* w, const int* pos,
                             const int* slots, int n, BbServeState* s, void* stream) {
  if (!c || !w || !s || li < 0 || li >= c->n_layers || n <= 0 || n > w->rows) return BB_EARG;
  return pre_attn(*c, li, *w, pos, slots, n, *s, stream);
}

BB_API int bb_serve_post_attn(const BbServeCfg* c, int li, const BbServeWork* w, int n,
                              BbServeState* s, void* stream) {
  if (!c || !w || !s || li < 0 || li >= c->n_layers || n <= 0 || n > w->rows) return BB_EARG;
  return post_attn(*c, li, *w, n, *s, stream);
}

// hn[n, d] = RMSNorm(x + delta) * norm_w  (the input of the LM head).
BB_API int bb_serve_finish(const BbServeCfg* c, const BbServeWork* w, const void* norm_w, void* hn,
                           int n, BbServeState* s, void* stream) {
  if (!c || !w || !s || !s->delta || n <= 0 || n > w->rows) return BB_EARG;
  // the sum x + delta is also written out (to the free residual buffer): the kernel then normalises
  // the bf16-rounded sum, exactly as every other residual step of the stack does
  void* xn = (s->x == w->xa) ? w->xb : w->xa;
  return bb_rmsnorm_fwd(s->delta, s->x, norm_w, hn, xn, w->rstd, n, c->d_model, c->eps, stream);
}

// One decode step for n sequences (one new token each): embedding, every layer with split-KV paged
// attention over the block tables, final norm.  seqlens[i] = pos[i] + 1.
BB_API int bb_serve_decode(const BbServeCfg* c, const BbServeWork* w, const void* tok_emb, int vocab,
                           const int* tokens, const int* pos, const int* slots,
                           const int* block_tables, int max_blocks, const int* seqlens,
                           const void* norm_w, void* hn, int n, BbServeState* s, void* stream) {
  if (!c || !w || !s || n <= 0 || n > w->rows || w->splits < 1) return BB_EARG;
  BB_TRY(bb_serve_begin(c, w, tok_emb, vocab, tokens, n, s, stream));
  const int qk_ld = (c->hq + c->hk) * c->hd;
  const float scale = 1.0f / sqrtf((float)c->hd);
  for (int li = 0; li < c->n_layers; ++li) {
    const BbServeLayer& L = c->layers[li];
    BB_TRY(pre_attn(*c, li, *w, pos, slots, n, *s, stream));
    if (c->kv_int8)
      BB_TRY(bb_paged_decode_i8(w->qk, qk_ld, L.kc, L.vc, L.ks, L.vs, block_tables, max_blocks,
                                seqlens, w->o, c->hq * c->hd, w->part_o, w->part_ml, n, c->hq, c->hk,
                                c->hd, c->block_size, w->splits, scale, stream));
    else
      BB_TRY(bb_paged_decode(w->qk, qk_ld, L.kc, L.vc, block_tables, max_blocks, seqlens, w->o,
                             c->hq * c->hd, w->part_o, w->part_ml, n, c->hq, c->hk, c->hd,
                             c->block_size, w->splits, scale, stream));
    BB_TRY(post_attn(*c, li, *w, n, *s, stream));
  }
  return bb_serve_finish(c, w, norm_w, hn, n, s, stream);
}
