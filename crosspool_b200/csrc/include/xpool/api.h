/* C ABI of libxpool_kernels.so. Every struct here is mirrored field-for-field by
 * a ctypes.Structure in crosspool_b200/native/__init__.py; bump XP_ABI_VERSION
 * when a layout changes (the Python side checks it at import, like the
 * reference checks its native ABI number, src/xpool/cext.py:1-30). */
#ifndef XPOOL_API_H_
#define XPOOL_API_H_

#include <stddef.h>
#include <stdint.h>

#define XP_ABI_VERSION 21

#ifdef __cplusplus
extern "C" {
#endif

typedef struct XpGemmArgs {
  const void* w;       /* [w_rows_total, k] bf16 weights (nn.Linear layout) */
  const void* x;       /* [rows, k] bf16 activations */
  void* out;           /* [rows, ld_out] */
  const void* resid;   /* optional [rows, ld_resid] bf16 */
  const float* bias;   /* optional fp32 per weight row */
  float* ws;           /* split-K workspace (optional) */
  uint32_t* counters;  /* split-K tile counters, zeroed once by the caller */
  uint32_t* status;    /* optional device word; first non-zero error code wins */
  void* stream;        /* cudaStream_t */
  size_t ws_bytes;
  size_t counter_bytes;
  int w_rows_total;    /* 0: derived from n_out / up_offset */
  int n_out;           /* features produced, multiple of 128 */
  int k;               /* multiple of 64 */
  int rows;
  int ldw, ldx, ld_out, ld_resid; /* element strides; 0 = dense */
  int epilogue;        /* 0 store bf16, 1 swiglu (dual), 2 residual add, 3 store fp32 */
  int dual;
  int up_offset;       /* first weight row of the up projection */
  int splits;          /* 0 = choose */
  int bn;              /* 0 = choose */
  int num_sms;         /* 0 = all */
  int w_evict_first;
  int w_tiled;         /* weights pre-tiled into contiguous 128x64 blocks */
  float gate_limit, up_add, act_alpha;
  /* grouped (MoE) form: device tile table of int4 {group, feature tile, first row, row end} */
  const void* tile_table;
  const int* n_tiles;
  int w_rows_per_group;
  int smem_limit;      /* > 0: cap on dynamic shared memory, so the CTA can share an SM with another stream's kernel */
  /* Block-scaled fp8: w and x are e4m3; w_scale [n_rows / 128][k / 128], x_scale [k / 128][ld_xscale] (fp32). */
  int fp8;
  const float* w_scale;
  const float* x_scale;
  int ld_xscale;
} XpGemmArgs;

typedef struct XpGemmPlan {
  size_t ws_bytes;
  size_t counter_bytes;
  int bn, nacc, splits, tiles, grid, smem_bytes, smem_budget, stages;
} XpGemmPlan;


/* Fused [wait partials] -> ordered sum -> (+residual) -> RMSNorm -> local store / peer push ->
 * release flags. One CTA per row. */
typedef struct XpNormArgs {
  const void* parts[8];        /* bf16 [rows, ld_parts] inputs summed in index order */
  const uint32_t* wait_flags[8]; /* optional, one per part: wait until >= wait_seq */
  void* out_peers[8];          /* bf16 [rows, ld_out] destinations (peer or local memory) */
  uint32_t* peer_flags[8];     /* sequence word released after all rows are stored */
  uint32_t* peer_meta[8];      /* optional 4-word invocation record written before the flag */
  void* resid;                 /* optional bf16 [rows, hidden], updated in place */
  const void* weight;          /* bf16 [hidden]; null = residual add only */
  void* out_local;             /* optional bf16 [rows, ld_out] */
  uint32_t* done_counter;      /* zeroed word used to find the last CTA */
  uint32_t* status;            /* optional error word */
  const uint32_t* cancel;      /* optional: non-zero aborts waits */
  uint64_t wait_ns;            /* wait limit */
  int rows, hidden, ld_parts, ld_out, nparts, npeers;
  uint32_t wait_seq, publish_seq, meta_layer, meta_mode, meta_deadline_us;
  float eps;
  uint32_t* seq_counter;       /* optional device word: publish value = *seq_counter + 1, stored back */
  const uint32_t* meta_deadline_ptr; /* optional device word overriding meta_deadline_us (refreshed per step) */
  /* observer (all null / 0: off) */
  void* trace_events;
  void* trace_state;
  uint32_t trace_capacity;
  uint32_t reserved;
} XpNormArgs;

/* Attention side: wait (bounded) until each flag reaches *want_ptr (or `want`). */
typedef struct XpWaitArgs {
  const uint32_t* flags[8];
  const uint32_t* want_ptr;
  const uint32_t* cancel;      /* usually the claim word of `failure`: non-zero ends the wait (status 5) */
  uint32_t* status;
  uint64_t wait_ns;
  uint32_t want;
  int n;
  /* Canonical failure: a wait that runs out claims `failure` (first failure wins) and copies it into the
     peers' slots so that every kernel waiting anywhere in the generation leaves at once. All optional. */
  void* failure;               /* local FailureSlot */
  void* peer_failures[8];      /* FailureSlots in the FFN ranks' memory */
  int n_peer_failures;
  uint32_t origin_pe, instance;
  /* observer (all null / 0: off) */
  void* trace_events;
  void* trace_state;
  uint32_t trace_capacity;
  uint32_t reserved;
} XpWaitArgs;

/* Producer half of a flag handshake: *seq_counter += 1, then every flag receives the new value (release). */
typedef struct XpSignalArgs {
  uint32_t* flags[8];
  uint32_t* seq_counter;
  int n;
  int reserved;
} XpSignalArgs;

/* Transport of one Instance rank of an external serving engine (see kernels/instance.cu). */
typedef struct XpInstanceBinding {
  void* peer_inputs[8];      /* FFN ranks: [capacity_rows, hidden] bf16 input buffers of the Instance's slots */
  void* peer_records[8];     /* FFN ranks: InvocationRecord of the slot */
  void* peer_flags[8];       /* FFN ranks: the record's sequence word */
  void* peer_failures[8];    /* FFN ranks: failure slot of the Instance's slot */
  const void* parts[8];      /* local: partial outputs of the FFN TP ranks, [capacity_rows, hidden] bf16 each */
  const void* done_flags[8]; /* local: completion sequence words, one per FFN TP rank */
  void* failure;             /* local failure slot (its claim word cancels the wait) */
  void* status;              /* device status word (4 timed out, 5 cancelled) */
  uint64_t wait_ns;          /* completion wait limit; 0: 5 s */
  int n_peers, n_parts, hidden, capacity_rows;
  uint32_t origin_pe, reserved;
} XpInstanceBinding;
int xp_instance_create(const XpInstanceBinding* b);
int xp_instance_set_current(int handle);
int xp_instance_current(void);
int xp_instance_submit(int handle, const void* hidden, int rows, int ld, void* out, int ld_out, int layer, int mode,
                       int requirement, int dp_layout, void* stream);
void xp_instance_destroy(int handle);

/* FFN device Lane runtime (see xpool/lane.cuh). */
typedef struct XpLaneInstanceDesc {
  void* input;             /* local [capacity_rows, hidden] bf16 payload buffer */
  void* act;               /* local [capacity_rows, act_ld] bf16 scratch */
  const void* in_flag;     /* local sequence word released by the attention side */
  const void* record;      /* local InvocationRecord */
  void* out_peer;          /* attention device: [capacity_rows, hidden] partial of this TP rank */
  void* done_record_peer;  /* attention device: CompletionRecord of this TP rank */
  int capacity_rows, hidden, num_layers, act_ld;
  void* failure_peer;      /* attention device: the Instance's failure slot (may be null) */
  int pe;                  /* this FFN device's PE number */
  int reserved;
} XpLaneInstanceDesc;

typedef struct XpLaneLayerDesc {
  const void* w_gateup;    /* [(gated ? 2 : 1) * inter_local, hidden] bf16 (row-major or tiled) */
  const void* w_down;      /* [hidden, inter_local] */
  const float* bias_gateup;
  const float* bias_down;
  int inter_local, gated, w_tiled;
  float gate_limit, up_add, act_alpha;
  /* Mixture of experts when num_experts > 0: w_gateup is [n_local * 2 * inter_local, hidden] and w_down
     [n_local * hidden, inter_local] for the experts [expert_lo, expert_hi) this rank owns. */
  const void* router;            /* [num_experts rounded up to 128, hidden] bf16, padding rows zero */
  const float* correction_bias;  /* optional [num_experts] */
  const float* router_bias;      /* optional [num_experts] */
  int num_experts, top_k, expert_lo, expert_hi, sigmoid, renormalize;
  float scale;
  int shared_inter_local;        /* > 0: shared experts as one dense gated FFN of this local width */
  const void* w_shared_gateup;   /* [2 * shared_inter_local, hidden] */
  const void* w_shared_down;     /* [hidden, shared_inter_local] */
  const void* router_raw;        /* [num_experts, hidden] weights of an fp32 router projection (bf16; fp32 if precision 2) */
  int router_precision;          /* 0 payload, 1 fp32 accumulate and logits from payload weights, 2 fp32 weights */
  int reserved;
} XpLaneLayerDesc;

void* xp_lane_create(int n_instances, int n_lanes, int policy, uint64_t seed, size_t ws_bytes_per_lane);
int xp_lane_set_instance(void* rt, int idx, const XpLaneInstanceDesc* d);
int xp_lane_set_layer(void* rt, int inst, int layer, const XpLaneLayerDesc* d);
int xp_lane_commit(void* rt);
int xp_lane_launch(void* rt, int lane_index, uint64_t lease_ns, void* stream);
int xp_lane_threads_start(void* rt, uint64_t lease_ns, int depth);
int xp_lane_threads_stop(void* rt);
int xp_lane_threads_state(void* rt, uint64_t* replays);
int xp_lane_shutdown(void* rt, void* stream);
int xp_lane_failure(void* rt, uint32_t out6[6], void* stream);   /* {claim, result, origin, instance, sequence, layer} */
/* Stand-alone event buffers for the attention-side observers (device memory). */
int xp_trace_create(uint32_t capacity, void** events, void** state);
int64_t xp_trace_read(void* events, void* state, uint32_t capacity, uint64_t* out, uint64_t max_events, uint64_t* dropped, void* stream);
void xp_trace_destroy(void* events, void* state);
int xp_lane_stats(void* rt, uint64_t* served, uint32_t* idle, uint32_t* status, void* stream);
int xp_lane_trace_enable(void* rt, uint32_t capacity);
int64_t xp_lane_trace_read(void* rt, uint64_t* out, uint64_t max_events, uint64_t* dropped, void* stream);
void xp_lane_destroy(void* rt);
int xp_wait_flags(const XpWaitArgs* a, void* stream);
int xp_signal_flags(const XpSignalArgs* a, void* stream);

/* Mixture-of-experts helpers (csrc/kernels/moe.cu). */
typedef struct XpRouterArgs {
  const void* logits;           /* [rows, ld_logits] bf16 or fp32 */
  const float* logit_bias;      /* optional [experts] added to the logits */
  const float* correction_bias; /* optional [experts] added to the scores for selection only */
  int* topk_ids;                /* [rows, top_k] */
  float* topk_weights;          /* [rows, top_k] */
  int rows, num_experts, top_k, ld_logits;
  int logits_fp32, sigmoid, renormalize, round_weights_bf16;
  float scale;
} XpRouterArgs;

typedef struct XpRouteArgs {
  const int* topk_ids;          /* [rows, top_k] */
  int* counts;                  /* [n_local] */
  int* offsets;                 /* [n_local + 1] */
  int* perm_token;              /* [rows * top_k] token of each ordered row */
  int* route_pos;               /* [rows * top_k] ordered row of each route, -1 if not local */
  void* tiles_gateup;           /* int4 tile table for the gate/up projection */
  void* tiles_down;
  int* n_tiles_gateup;
  int* n_tiles_down;
  int rows, top_k, expert_lo, expert_hi;
  int tm_gateup, bn_gateup, tm_down, bn_down;
} XpRouteArgs;

int xp_router_topk(const XpRouterArgs* a, void* stream);
/* Router projection with IEEE fp32 accumulation: x bf16 [rows, ldx], w [experts, hidden] bf16 (w_fp32 = 0) or fp32. */
int xp_router_fp32(const void* x, int ldx, const void* w, int w_fp32, float* logits, int ld_logits, int rows, int hidden,
                   int num_experts, void* stream);
int xp_moe_route(const XpRouteArgs* a, void* stream);
int xp_moe_gather(const void* x, const int* perm_token, const int* n_rows_ptr, void* out, int max_rows,
                  int hidden, int ldx, void* stream);
int xp_moe_combine(const void* y, const int* route_pos, const float* weights, void* out, int rows, int top_k,
                   int hidden, int ld_out, void* stream);

/* Raw device memory shared between processes (CUDA IPC). */
int xp_dev_alloc(void** ptr, size_t bytes);
int xp_dev_free(void* ptr);
int xp_ipc_get_handle(void* ptr, void* handle64);
int xp_ipc_open(const void* handle64, void** ptr);
int xp_ipc_close(void* ptr);
int xp_memset_async(void* ptr, int value, size_t bytes, void* stream);
int xp_enable_peer_access(int peer_device);

int xp_norm_publish(const XpNormArgs* a, void* stream);
int xp_swiglu(const void* gate_up, void* out, int rows, int inter, float limit, float up_add,
              float alpha, void* stream);

/* q/k RMSNorm + rotary embedding + paged KV scatter over a fused QKV projection. */
typedef struct XpRopeArgs {
  const void* qkv;            /* bf16 [rows, ld_qkv]: q heads, k heads, v heads */
  void* q_out;                /* bf16 [rows, q_heads, head_dim] */
  void* k_cache;              /* bf16 [pages, page_size, kv_heads, head_dim] */
  void* v_cache;
  const void* q_norm_weight;  /* optional bf16 [head_dim] */
  const void* k_norm_weight;
  const int* positions;       /* [rows] */
  const int* slots;           /* [rows] page * page_size + offset, -1 = skip */
  int rows, ld_qkv, q_heads, kv_heads, head_dim;
  float eps, log2_theta;
} XpRopeArgs;

typedef struct XpDecodeAttnArgs {
  const void* q;              /* bf16 [batch, q_heads, head_dim] */
  const void* k_cache;
  const void* v_cache;
  void* out;                  /* bf16 [batch, q_heads, head_dim] */
  float* ws;                  /* [batch, q_heads, splits, head_dim + 2] when splits > 1 */
  const int* block_table;     /* [batch, max_blocks] */
  const int* seq_lens;        /* [batch] tokens in cache including the current one */
  int batch, q_heads, kv_heads, head_dim, page_size, max_blocks, num_splits;
  float scale;
  int chunk_tokens;           /* > 0: slices of this many tokens (num_splits = ceil(max_len / chunk)) */
  int num_pages;              /* pages in the cache (bound of the tensor maps); 0: SIMT kernel only */
  uint32_t* status;           /* optional: set non-zero when a bounded wait ran out */
  int force_simt;             /* testing: skip the tensor-core kernel */
  int reserved;
} XpDecodeAttnArgs;

typedef struct XpPrefillAttnArgs {
  const void* q;              /* bf16 [total_q, q_heads, head_dim], sequences packed */
  const void* k_cache;
  const void* v_cache;
  void* out;                  /* bf16 [total_q, q_heads, head_dim] */
  const int* block_table;     /* [num_seqs, max_blocks] */
  const int* q_starts;        /* [num_seqs] first packed row of the chunk */
  const int* q_lens;          /* [num_seqs] rows in the chunk */
  const int* ctx_lens;        /* [num_seqs] tokens cached before the chunk */
  int num_seqs, max_q_len, q_heads, kv_heads, head_dim, page_size, max_blocks;
  float scale;
  int num_pages;              /* pages in the cache (bound of the tensor maps); 0: simple kernel only */
  int force_simple;           /* kernel choice: 0 tcgen05 kernel (falls back when the shape is outside it),
                                 1 plain mma.sync kernel, 2 TMA-fed mma.sync kernel; bit 8: the tcgen05 kernel stages
                                 the probabilities in shared memory instead of tensor memory */
  uint32_t* status;           /* optional, FOUR words: [0] set non-zero when a bounded wait ran out (7: tcgen05 kernel),
                                 [1..3] detail of the first such CTA (wait site, block, tiles) */
  int total_q;                /* rows of q / out (bound of the query tensor map); 0: no tcgen05 kernel */
} XpPrefillAttnArgs;

int xp_rope_kv(const XpRopeArgs* a, void* stream);
int xp_decode_attn_splits(int batch, int kv_heads, int max_len);
int xp_decode_attn(const XpDecodeAttnArgs* a, void* stream);
int xp_prefill_attn(const XpPrefillAttnArgs* a, void* stream);
int xp_prefill_attn_umma(const XpPrefillAttnArgs* a, void* stream);

/* Small row-wise helpers. */
int xp_embedding(const int* ids, const void* table, void* out, int rows, int hidden, int vocab,
                 void* stream);
int xp_argmax(const void* logits, int is_fp32, int* out, int rows, int vocab, int ld, void* stream);
int xp_sample(const void* logits, int is_fp32, const float* temps, const uint32_t* seeds, int* out, int rows, int vocab,
              int ld, void* stream);
int xp_fill_u32(void* p, uint32_t v, size_t n, void* stream);
int xp_l2_flush(void* p, size_t bytes, void* stream);

int xp_abi_version(void);
/* device mirror of the process's debug options: transport, fabric, graph, routing observer switches */
int xp_debug_options_set(const uint32_t* four);
int xp_debug_options_get(uint32_t* four);
int xp_gemm_plan(const XpGemmArgs* a, XpGemmPlan* plan);
int xp_quant_act_fp8(const void* x, void* xq, float* scales, int rows, int k, int ldx, int ldq, int ld_scale, void* stream);
int xp_gemm(const XpGemmArgs* a);
int xp_encode_tmap_2d(void* out128, const void* base, uint64_t rows, uint64_t cols,
                      uint64_t pitch_bytes, uint32_t box_rows, uint32_t elem_bytes);

#ifdef __cplusplus
}
#endif
#endif /* XPOOL_API_H_ */
