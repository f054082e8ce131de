// Plain-C structures that cross the library boundary (decode engine descriptors, GEMM staging request).
// prometorch_b200/_native.py mirrors them with ctypes; keep the two in step.
#pragma once

#define PTB_MAX_PEERS 8

// One quantised matrix in the layout its kernel streams.
typedef struct PtbWeightDesc {
    const void* w;          // a GEMV streaming layout (see `layout`) or, for tables, row-major rows
    const void* bias;       // optional fp32 [rows]
    int qtype;              // 0 = Q4_K, 1 = Q6_K (structure of arrays), tables also: 2 = fp16, 3 = fp32
    int rows, cols;
    int rowbytes;           // > 0 only for row-major tables (the embedding)
    int layout;             // 0: [segment][row][segment bytes] (dp4a kernel); 1: tiles of 16 rows (tensor-pipe kernel)
    int pad;
} PtbWeightDesc;

typedef struct PtbLayerDesc {
    PtbWeightDesc q, k, v, o, gate, up, down;
    const float* attn_norm;
    const float* ffn_norm;
    const float* q_norm;
    const float* k_norm;
    const float* cos;       // per-layer RoPE tables [max_seq][head_dim / 2] (sliding-window layers may use another base)
    const float* sin;
    int window;             // sliding-window width, 0 = full attention
    int pad;
    const float* post_attn_norm;   // RMSNorm of the attention block's output before the residual add (or null)
    const float* post_ffn_norm;    // ... and of the FFN block's output
} PtbLayerDesc;

typedef struct PtbModelDesc {
    int n_layers, hidden, n_heads, n_kv_heads, head_dim, inter, vocab, max_seq;   // head counts are per rank
    float eps, emb_scale;
    int neox, act_gelu, norm_add_one, want_logits;
    PtbWeightDesc embed, lm_head;
    const float* out_norm;
    int tp_rank, tp_world, vocab_offset, pad;
    void* peer_inbox[3][PTB_MAX_PEERS];     // tensor parallelism: three receive buffers (attention out, FFN down, lm_head pair)
    int slot_elems, pad2;
} PtbModelDesc;

// Request to stage a row-sharded GEMM operand from the peers inside the launch.
typedef struct PtbStaging {
    void* peer[PTB_MAX_PEERS];   // peer r's full-size buffer as mapped on this GPU
    void* local;                 // this GPU's full-size buffer
    void* flags;                 // uint32 [ceil(stored_rows / 128)]: last sequence number staged per 128-row block
    int rank, world, shard_rows, stored_rows;
    long long row_bytes;
    unsigned seq;                // 0 disables staging
    int external;                // non-zero: someone else (copy engines on a side stream) copies the rows and raises the
                                 // flags; the launch adds no stager CTAs and only waits on the flags
} PtbStaging;

// One request of ptb_sample_logits_batch: a row of fp32 logits, the request's id history (the chosen id is appended at
// history[n_hist] when it fits), its scratch (ptb_sample_scratch_bytes, zeroed once) and where the result goes
// (out[0] = id, out[1] = float bits of its probability).  `u` is the uniform number of the draw.
typedef struct PtbSampleRequest {
    const float* logits;
    int* history;
    void* scratch;
    int* out;
    int n_hist, hist_cap, top_k, pad;
    float repeat_penalty, temperature, top_p, u;
} PtbSampleRequest;
