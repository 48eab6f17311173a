/*
 * promptcache_b200 -- C ABI of the sequence-batch kernels (libpromptcache_b200_seq.so).
 *
 * These kernels serve models whose step runs a BATCH of sequences as one concatenated token matrix over a pool of
 * per-sequence slots: attention layers keep K/V rows per slot, recurrent layers keep a state per slot.  Each mechanism
 * is one entry point whose constants are parameters, so that several model designs can share them:
 *
 *   pcs_embed            token embedding times a scale into the 32-bit residual stream
 *   pcs_rmsnorm          RMS norm of 32-bit rows, result in the compute type
 *   pcs_gate_norm_add    x += ls * w * rms(y * sigmoid(g))   (gated sublayer result, output norm, layer scale, residual sum),
 *                        optionally followed by the next sublayer's input norm
 *   pcs_xielu            xIELU activation
 *   pcs_qk_prep          whole-projection RMS norm of q and k, position-dependent query temperature, value mixing with an
 *                        earlier layer's values, append of K/V rows to the slot pool
 *   pcs_attn             causal attention over the slot pool with distinct key and value widths, grouped heads, an optional
 *                        logarithmic distance bias and an optional sink term in the softmax denominator
 *   pcs_mlstm_gates      capped input / forget gate pre-activations of a matrix-memory recurrent layer
 *   pcs_mlstm_scan       the stabilised matrix-memory recurrence with its per-head output norm and output gate
 *
 * All tensor arguments are DEVICE pointers; `dtype` selects the compute / storage type of activations, weights and K/V
 * rows: PCS_BF16 or PCS_F32 (true 32-bit everywhere).  The residual stream, norms' statistics, attention scores and
 * weights, gates and recurrent state are 32-bit floats in both modes.  Calls are asynchronous on `stream`.
 *
 * The batch is described by int32 arrays on the device:
 *   tok_seq[t]   batch entry of token t          tok_pos[t]   position of token t inside its sequence
 *   seq_slot[b]  pool slot of entry b            seq_pos0[b]  rows / tokens the slot already holds
 *   seq_len[b]   new tokens of entry b           seq_off[b]   index of its first token in the concatenated matrix
 */
#ifndef PROMPTCACHE_B200_SEQ_H_
#define PROMPTCACHE_B200_SEQ_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCS_ABI_VERSION 1
#define PCS_BF16 0
#define PCS_F32 1

enum { PCS_OK = 0, PCS_ERR_INVALID = -1, PCS_ERR_UNSUPPORTED = -2, PCS_ERR_CUDA = -3 };

int pcs_version(void);
const char* pcs_last_error(void);
int64_t pcs_launch_count(void);

/* out[t, :] = table[ids[t], :] * scale        (out fp32 [n, width]; ids int64) */
int pcs_embed(const void* table, const int64_t* ids, float* out, int n_tokens, int width, int vocab, float scale, int dtype,
              void* stream);

/* out[r, :] = x[rows ? rows[r] : r, :] / sqrt(mean(x^2) + eps) * w      (x fp32, w and out in `dtype`) */
int pcs_rmsnorm(const float* x, const int32_t* rows, const void* w, void* out, int n_rows, int width, float eps, int dtype,
                void* stream);

/* x[r, :] += ls * w * rms(y[r, :] * sigmoid(g[r, :]))   (g may be NULL: no gate; ls may be NULL: no layer scale)
 * then, if next_w != NULL, h_out[r, :] = rms(x[r, :]) * next_w.  y and g are `dtype` with row strides in elements. */
typedef struct pcs_gna_params {
  float* x;
  const void* y;
  const void* g;
  int64_t y_stride, g_stride;
  const void* w;
  const void* ls;
  const void* next_w;
  void* h_out;
  int n_rows, width;
  float eps;
  int dtype;
} pcs_gna_params;
int pcs_gate_norm_add(const pcs_gna_params* p, void* stream);

/* xIELU: z > 0: softplus(a[0]) z^2 + z/2;  z <= 0: (1/2 + softplus(a[1])) (exp(z) - 1 - z) + z/2.   `a` holds two `dtype` numbers. */
int pcs_xielu(const void* z, int64_t z_stride, void* out, int64_t out_stride, const void* a, int n_rows, int width, int dtype,
              void* stream);

typedef struct pcs_qkprep_params {
  const void* qkv;          /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off (biases already added) */
  int64_t row_stride;
  int32_t q_off, k_off, v_off;
  const void* q_norm_w;     /* [H*dim] or NULL (no query norm) */
  const void* k_norm_w;     /* [Hkv*dim] or NULL */
  float eps;
  int32_t n_heads, n_kv_heads, dim, vdim;
  float temp_coef;          /* q *= 1 + temp_coef * ln(floor((pos + 1) / temp_every) + 1); temp_every <= 0: none */
  int32_t temp_every;
  void* q_out;              /* [n_tokens, H*dim] */
  void* k_pool;             /* [slots, Hkv, cap, dim] */
  void* v_pool;             /* [slots, Hkv, cap, vdim] */
  int32_t cap;
  const void* v_first_pool; /* value pool of the layer whose values are mixed in, or NULL */
  const void* v_lambda;     /* one `dtype` number: v = (1 - lambda) v + lambda v_first */
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  int32_t n_tokens, dtype;
} pcs_qkprep_params;
int pcs_qk_prep(const pcs_qkprep_params* p, void* stream);

typedef struct pcs_attn_params {
  const void* q;            /* [n_tokens, H*dim] */
  const void* k_pool;
  const void* v_pool;
  void* out;                /* [n_tokens, H*vdim] */
  int32_t n_heads, n_kv_heads, dim, vdim, cap;
  float scale;
  const float* bias_r1;     /* [H] or NULL: score -= r1[h] * ln(1 + r2[h] * (i - j)) */
  const float* bias_r2;
  int32_t sink;             /* 1: softmax denominator has one more term exp(0) that carries no value */
  const int32_t* tok_seq;
  const int32_t* tok_pos;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_tokens, n_seqs, max_len, dtype;   /* max_len: host upper bound of the new tokens of one entry */
  int32_t impl;             /* 0 = automatic, 1 = the plain kernel */
  int32_t max_keys;         /* host upper bound of the keys one token sees (sizes the split of the keys); 0: one split */
  float* workspace;         /* fp32 scratch of pcs_attn_workspace_floats() elements, or NULL (one split) */
  int64_t workspace_floats;
} pcs_attn_params;
/* scratch the key split of pcs_attn needs for n_tokens tokens */
int64_t pcs_attn_workspace_floats(int n_tokens, int n_heads, int vdim);
int pcs_attn(const pcs_attn_params* p, void* stream);

/* ig = cap * tanh((w_i h + b_i) / cap);  fg = logsigmoid(cap * tanh((w_f h + b_f) / cap))    (fp32 [n_tokens, heads]) */
int pcs_mlstm_gates(const void* h, int64_t h_stride, const void* w_i, const void* w_f, const float* b_i, const float* b_f,
                    float* ig, float* fg, int n_tokens, int width, int heads, float cap, int dtype, void* stream);

/* out[m, n] = sum_k x[m, k] w[n, k] + bias[n] for 1 to 8 rows (decoding): the weights are streamed once, sums are fp32.
   k, the row stride of x and the pointers of x and w must be multiples of 16 bytes. */
int pcs_linear_rows(const void* x, int64_t x_stride, const void* w, const void* bias, void* out, int64_t out_stride, int m, int n, int k,
                    int dtype, void* stream);

typedef struct pcs_mlstm_params {
  const void* proj;         /* [n_tokens, row_stride]: q at q_off, k at k_off, v at v_off, output-gate pre-activation at g_off */
  int64_t row_stride;
  int32_t q_off, k_off, v_off, g_off;
  const float* ig;          /* [n_tokens, heads] log input gate  */
  const float* fg;          /* [n_tokens, heads] log forget gate */
  const void* norm_w;       /* [heads*vdim] */
  void* out;                /* [n_tokens, heads*vdim] */
  float* s_pool;            /* [slots, heads, dim, vdim] */
  float* n_pool;            /* [slots, heads, dim] */
  float* m_pool;            /* [slots, heads] */
  int32_t heads, dim, vdim;
  float q_scale;            /* dim^(-1/2) */
  float eps;
  const int32_t* seq_slot;
  const int32_t* seq_pos0;
  const int32_t* seq_len;
  const int32_t* seq_off;
  int32_t n_seqs, dtype;
  int32_t max_len;          /* host upper bound of the new tokens of one entry */
  int32_t impl;             /* 0 = automatic, 1 = token by token with the state in shared memory, 2 = token by token (registers
                               where the sizes allow): never the chunkwise tensor-core kernel */
  float* o_raw;             /* fp32 scratch of n_tokens*heads*vdim + n_seqs*heads*(dim+1) elements: the recurrence's result before
                               the per-head norm, and the new n / m of every entry until they are committed */
  int32_t n_tokens, reserved;
} pcs_mlstm_params;
int pcs_mlstm_scan(const pcs_mlstm_params* p, void* stream);

#ifdef __cplusplus
}
#endif
#endif
