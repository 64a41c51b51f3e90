/* kllm_seq.h -- C-ABI of the sequence-batch engine of kuiperllama_b200 (sm_100a).
 *
 * The single-sequence decoder of kllm_b200.h runs one position of one sequence per step.  This engine runs a STEP
 * of several sequences at once: every entry of a step brings the next tokens of one sequence (a whole prompt, or one
 * decoded token), all tokens of the step go through the layers as one ragged batch (no padding), and the keys and
 * values of every sequence live in fixed-size pages of one pool that sequences take as they grow and give back when
 * they end.  The layer stack is described by data (kllm_seq_layer), not by a model class: pre/post layer norms around
 * a token mixer and around a feed-forward, a schedule that may run a span of layers several times with the same
 * weights (each run with a cache of its own), so other model families can be described with the same pieces.
 *
 * Numerics.  compute type KLLM_SEQ_F32: every product in true fp32.  KLLM_SEQ_BF16: matrix products read bf16 weights
 * and bf16 activations and accumulate in fp32; keys / values are cached in bf16.  In both, the residual stream, the
 * norms, attention scores and softmax weights, the router and all gates are fp32.
 *
 * Same conventions as kllm_b200.h: device pointers in the descriptor, return 0 = ok, > 0 cudaError_t, < 0 KLLM_E_*.
 */
#ifndef KLLM_SEQ_H_
#define KLLM_SEQ_H_
#include "kllm_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

#define KLLM_SEQ_F32 0
#define KLLM_SEQ_BF16 1

#define KLLM_SEQ_MIXER_ATTENTION 1 /* softmax attention over the sequence's cached keys */
#define KLLM_SEQ_FF_NONE 0
#define KLLM_SEQ_FF_MOE 1 /* softmax router, top-k SwiGLU experts, optional gated shared expert */

typedef struct kllm_seq_norm {
  const float* w; /* [width] */
  const float* b; /* [width] or NULL */
} kllm_seq_norm;

typedef struct kllm_seq_attention {
  int32_t heads, kv_heads, dim, vdim; /* query heads, key/value heads, query-key size, value size per head */
  float scale;                        /* score = (q . k) * scale */
  float temp_coef;                    /* query temperature 1 + coef * ln(floor((pos + 1) / every) + 1) ... */
  int32_t temp_every;                 /* ... 0: none */
  int32_t qk_norm;                    /* RMS norm over dim of each query / key head, weights below */
  int32_t gate;                       /* sigmoid output gate per (token, head); its rows close w_in */
  const void* w_in;  /* [heads*dim + kv_heads*dim + kv_heads*vdim (+ heads), width]: q | k | v (| gate) rows, compute type */
  const float* q_norm_w; /* [dim] */
  const float* k_norm_w; /* [dim] */
  const void* w_out;     /* [width, heads*vdim], compute type */
} kllm_seq_attention;

typedef struct kllm_seq_moe {
  int32_t experts, top, ff; /* routed experts, chosen per token, inner size of a routed expert */
  float router_scale;       /* weights = chosen softmax scores / (their sum + 1e-20) * router_scale */
  const float* w_router;    /* [experts, width] fp32 */
  const void* gate_up;      /* [experts][2*ff][width]: gate rows, then up rows; compute type */
  const void* down;         /* [experts][width][ff] */
  int32_t shared_ff;        /* 0: no shared expert */
  const void* shared_gate_up; /* [2*shared_ff][width] */
  const void* shared_down;    /* [width][shared_ff] */
  const float* w_shared_gate; /* [width] fp32: the shared expert's output is scaled by sigmoid(w . h); NULL: by 1 */
} kllm_seq_moe;

typedef struct kllm_seq_layer {
  int32_t mixer_kind; /* KLLM_SEQ_MIXER_* */
  int32_t ff_kind;    /* KLLM_SEQ_FF_* */
  /* x += post_mixer(mixer(pre_mixer(x)));  x += post_ff(ff(pre_ff(x))) */
  kllm_seq_norm pre_mixer, post_mixer, pre_ff, post_ff;
  kllm_seq_attention attn;
  kllm_seq_moe moe;
} kllm_seq_layer;

typedef struct kllm_seq_desc {
  int32_t dtype; /* KLLM_SEQ_F32 / KLLM_SEQ_BF16 */
  int32_t width, vocab;
  float norm_eps;
  int32_t n_layers;
  const kllm_seq_layer* layers;
  /* the order in which layers run: run r executes layer run_layer[r] with cache r; run_add[r] >= 0 adds row
   * run_add[r] of `run_vectors` ([*, width] fp32) to the residual stream right before it */
  int32_t n_runs;
  const int32_t* run_layer;
  const int32_t* run_add;
  const float* run_vectors;
  const void* embed; /* [vocab, width] compute type */
  kllm_seq_norm final_norm;
  const void* head;  /* [vocab, width] compute type */
  /* cache geometry */
  int32_t max_tokens; /* tokens all live sequences may hold together */
  int32_t max_seqs;   /* live sequences */
  int32_t page_tokens; /* tokens per page; 0: the engine's default */
} kllm_seq_desc;

typedef struct kllm_seq_engine kllm_seq_engine;

int kllm_seq_create(const kllm_seq_desc* desc, void* stream, kllm_seq_engine** out);
void kllm_seq_destroy(kllm_seq_engine* eng);

/* Sequences: open returns a slot; close gives its pages back to the pool. */
int kllm_seq_open(kllm_seq_engine* eng, int32_t* seq_out);
int kllm_seq_close(kllm_seq_engine* eng, int32_t seq);
int kllm_seq_length(const kllm_seq_engine* eng, int32_t seq);
int kllm_seq_free_pages(const kllm_seq_engine* eng);

/* One step.  Entry e appends counts[e] tokens (tokens_host, concatenated in entry order) to sequence seqs[e].
 * want_host lists the rows (indices into the concatenated tokens) whose logits are wanted; they are written to
 * logits_host [n_want, vocab] (fp32) and, when argmax_host is given, their greedy ids to argmax_host [n_want].
 * Blocking: returns after the results are in host memory. */
int kllm_seq_step(kllm_seq_engine* eng, int32_t n_entries, const int32_t* seqs, const int32_t* counts,
                  const int32_t* tokens_host, int32_t n_want, const int32_t* want_host, float* logits_host,
                  int32_t* argmax_host);

/* Diagnostics: the next step also copies the residual stream after every layer run to host memory
 * [n_runs, tokens of the step, width]; fusions across layer runs are switched off for that step. */
int kllm_seq_trace_residual(kllm_seq_engine* eng, float* residual_host);
/* Measurement aid: the next step records an event after each of its phases and writes the device time spent in every
 * phase class, in milliseconds, to phase_ms[KLLM_SEQ_PHASES] (summed over the layer runs). */
#define KLLM_SEQ_PHASE_NORM 0       /* embedding rows, residual + layer-norm kernels */
#define KLLM_SEQ_PHASE_IN_PROJ 1    /* q | k | v | gate product */
#define KLLM_SEQ_PHASE_QK_PREPARE 2 /* head norms, temperature, cache scatter, gates */
#define KLLM_SEQ_PHASE_ATTENTION 3  /* paged attention + merge of the key splits */
#define KLLM_SEQ_PHASE_OUT_PROJ 4
#define KLLM_SEQ_PHASE_ROUTER 5     /* residual + norms around the router and the router itself (one kernel) */
#define KLLM_SEQ_PHASE_EXPERTS 6    /* routed experts */
#define KLLM_SEQ_PHASE_SHARED 7     /* shared expert */
#define KLLM_SEQ_PHASE_HEAD 8       /* final norm of the wanted rows, classifier, argmax, copies */
#define KLLM_SEQ_PHASES 9
int kllm_seq_profile(kllm_seq_engine* eng, float* phase_ms);
/* kernel launches of the last step */
int kllm_seq_last_launches(const kllm_seq_engine* eng);

/* The engine's token-block product on its own: out[T, N] (fp32) = a[T, K] . w[N, K]^T with a and w in the compute
 * type `dtype` (device pointers).  Picks the kernel the engine would pick for this shape. */
int kllm_seq_gemm(int32_t dtype, const void* a, const void* w, float* out, int32_t n_tokens, int32_t in_dim,
                  int32_t out_dim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KLLM_SEQ_H_ */
