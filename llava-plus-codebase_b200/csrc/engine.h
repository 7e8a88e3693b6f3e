// Engine objects behind the C ABI handles (b2_model, b2_kv) and the helpers the engine files share.
// model.cu owns the LLaVA path (ViT, projector, LLaMA decoder); seq_engine.cu owns decoders described by a list of layers.
#pragma once
#include <cuda_runtime.h>

#include <mutex>
#include <string>
#include <vector>

#include "../../include/b2llava.h"
#include "common.cuh"
#include "kernels.h"

namespace b2 {
typedef __nv_bfloat16 bf16;

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
    int alloc(size_t n) {
        free();
        if (n == 0) return 0;
        cudaError_t e = cudaMalloc(&p, n);
        if (e != cudaSuccess) {
            p = nullptr;
            set_error("cudaMalloc(%zu bytes) failed: %s", n, cudaGetErrorString(e));
            return -2;
        }
        bytes = n;
        return 0;
    }
    void free() {
        if (p) cudaFree(p);
        p = nullptr;
        bytes = 0;
    }
    template <typename T>
    T* as() const { return reinterpret_cast<T*>(p); }
};

struct VitLayer {
    DevBuf ln1_g, ln1_b, wqkv, bqkv, wo, bo, ln2_g, ln2_b, w1, b1, w2, b2;
    unsigned qkv_w = 0, qkv_b = 0;  // bit j set: part j (q/k/v) of the fused buffer has arrived
};
struct LlamaLayer {
    DevBuf ln1, wqkv, wo, ln2, wgu, wd;
    unsigned qkv_parts = 0;
    DevBuf wqkv8, wo8, wgu8, wd8, s_qkv, s_o, s_gu, s_d;  // e4m3 copies + per-row fp32 scales (b2_model_enable_fp8_decode)
    DevBuf tmp_gate, tmp_up;  // staging until both halves arrived
    bool has_gate = false, has_up = false;
};
// makes `dev` current for the duration of an ABI call and restores the caller's device afterwards
struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) prev = -1;
        if (prev != dev) cudaSetDevice(dev); else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
    DeviceGuard(const DeviceGuard&) = delete;
    DeviceGuard& operator=(const DeviceGuard&) = delete;
};

struct SeqModel;  // layer-list decoder (seq_engine.cu)
struct SeqState;  // its per-cache recurrent state and key/value slabs
}  // namespace b2

struct b2_model {
    typedef b2::DevBuf DevBuf;
    b2_model_desc d;
    int arch = 0;                  // B2_ARCH_LLAVA | B2_ARCH_LAYER_LIST
    b2::SeqModel* seq = nullptr;   // B2_ARCH_LAYER_LIST: layer descriptions, weights, workspaces (seq_engine.cu)
    int device = 0;
    std::mutex mu;
    bool finalized = false;
    // derived
    int P = 0, T = 0, kpad = 0, vit_live = 0, vit_hd = 64, hd = 128;
    // weights
    DevBuf patch_w, cls, pos, pre_g, pre_b;
    std::vector<b2::VitLayer> vit;
    DevBuf p0_w, p0_b, p2_w, p2_b;
    DevBuf embed, final_norm, lm_head;
    std::vector<b2::LlamaLayer> ll;
    // errors detected by kernels (bad token ids / image rows): int[8] in mapped pinned host memory, slot = log2(B2_ERR_*)
    int* err_host = nullptr;
    int* err_dev = nullptr;
    // the workspaces below are shared by every call on this model: a call on stream B must not start before the previous
    // call's kernels on stream A are done with them (calls on one stream are ordered anyway)
    cudaEvent_t ws_event = nullptr;
    cudaStream_t ws_stream = nullptr;
    bool ws_valid = false;
    // ViT workspace (per chunk of max_images)
    DevBuf v_col, v_patch, v_hidden, v_xn, v_qkv, v_attn, v_mlp, v_feats, p_mid, p_done;
    // LLaMA workspace
    DevBuf x, xn, qkv, attn, act, last_idx, xlast, logits, splice_idx;
    // encode_images replays a CUDA graph per chunk size (~190 launches per image, 5-20 us each at B = 1: the host cannot
    // keep the GPU fed launch by launch). Inputs/outputs are staged through fixed buffers so the captured pointers stay valid.
    DevBuf enc_pixels, enc_out;
    std::vector<cudaGraphExec_t> enc_graph;  // index = images in the chunk (0 = unused)
    std::vector<char> enc_warm;              // an eager run has set the function attributes for this chunk size
    cudaStream_t enc_stream = nullptr;       // capture is illegal on the legacy default stream: such callers run here
    cudaEvent_t enc_fork = nullptr, enc_join = nullptr;
    int enc_launches = 0;                    // kernels in one captured chunk (b2_launch_count bookkeeping)
    // fp8 decode (BASELINE configs[4]): e4m3 lm_head + scales, quantised activation row buffer + per-token scales
    bool fp8_decode = false;
    DevBuf lm_head8, s_head, xq8, xscale;
};

struct b2_kv {
    typedef b2::DevBuf DevBuf;
    b2_model* m = nullptr;
    b2::SeqState* seq = nullptr;   // B2_ARCH_LAYER_LIST: per-slot recurrent state, convolution tails, key/value slabs
    int seq_graph_launches = 0;    // kernels in the captured decode step of a layer-list model
    int max_batch = 0, max_seq = 0;
    DevBuf k, v;  // [L][B][H][Smax][D]
    DevBuf len_dev, tok, step_counter, out_tokens, attn_partial, attn_counters;
    DevBuf sk_partial, sk_counters;  // stream-K workspace of the skinny decode GEMM (batch 9..128)
    std::vector<int32_t> len_host;
    int out_capacity = 0;  // steps
    // cached decode-step graph
    cudaGraphExec_t graph = nullptr;
    int graph_B = 0;
    // stream capture is illegal on the legacy default stream (torch's default current stream): decode steps
    // run on this library-owned stream, ordered against the caller's stream with events
    unsigned int mega_bar_base = 0;  // value of the grid-barrier counter before the next megakernel launch
    DevBuf mega_layers, mega_sync;  // MegaLayer[L] table and {bar_count, bar_gen, done_count}
    DevBuf rope_tab;                // uint32 [max_seq][hd/2]: bf16 (cos, sin) per position for the QKV GEMM's fused RoPE epilogue
    cudaStream_t own_stream = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    int warm_B = 0;  // an eager step has run for this B (function attributes set, driver entry points resolved)
    // token selection state (sampling.cu) + the host-visible token ring of the streaming decode API
    DevBuf sstate;                 // SampleState on the device
    b2::SampleState samp_host = {};    // what was last written there (pub_counter / done excluded: the device advances them)
    bool samp_valid = false;
    int32_t* ring_host = nullptr;  // cudaHostAlloc(mapped) [ring_cap][max_batch]; entry = tag << 20 | token
    int32_t* ring_dev = nullptr;
    int ring_cap = 0;
    int epoch = 0;                 // generations started on this cache (tag = 1 + epoch % 2047)
    int stream_B = 0, stream_tag = 0, stream_scheduled = 0;  // streaming generation in progress: tokens scheduled so far
    DevBuf rows_dev;               // RowState[max_batch] (continuous batching)
    std::vector<b2::RowState> rows_host;
    size_t layer_stride() const { return (size_t)max_batch * m->d.heads * max_seq * m->hd; }
};


namespace b2 {
// Cross-stream ordering of the shared model workspaces (see b2_model::ws_event). Caller holds the model lock.
int ws_enter(b2_model* m, cudaStream_t st);
int ws_leave(b2_model* m, cudaStream_t st);
// what every b2_kv has, whatever the model: slot lengths, token feedback, step counter, selection state, host token ring
int kv_alloc_common(b2_kv* kv);
// error flags in mapped host memory and the workspace event of a model (b2_model_finalize)
int model_common_init(b2_model* m);
// layer-list decoders (seq_engine.cu)
int seq_set_weight(b2_model* m, const char* key, const void* ptr, const int64_t* shape, int ndim, int dtype);
int seq_finalize(b2_model* m);
void seq_model_free(b2_model* m);
int seq_kv_alloc(b2_kv* kv);
void seq_kv_free(b2_kv* kv);
int seq_decode_launch(b2_model* m, b2_kv* kv, int B, int slot0, cudaStream_t st);
}  // namespace b2
