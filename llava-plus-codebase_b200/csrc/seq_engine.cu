// Layer-list decoders behind the b2_model / b2_kv handles (include/b2llava.h, "layer-list decoders"): weights by tensor
// name, per-slot recurrent state and key/value slabs, and ONE forward over a set of rows that serves prompt portions
// (b2_append_tokens: n rows of one slot) and decode steps (one row per slot, replayed from the cache's CUDA graph by
// model.cu's decode_step_run with the same token selection and publication as the LLaMA path).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <map>

#include "engine.h"

namespace b2 {

struct SeqWeights {   // tensors of one layer that owns its weights
    // Linear weights in the compute dtype ([out, in]); vectors and small tables fp32
    DevBuf norm1, norm1_b, norm2, norm2_b;
    DevBuf in_w, conv_w, conv_b, dt_bias, a_log, skip, mnorm, o_w;                       // mamba2
    DevBuf lproj_w, rel, lo_w;                                                           // attention: [q | k | v | g] fused
    DevBuf mu, r_w, k_w, v_w, g_w, w1, w2, w0, bonus, rnorm, ro_w;                       // RWKV
    DevBuf up_w, down_w;                                                                 // feed-forward
    std::map<std::string, int> got;
};

struct SeqLayerInfo {
    b2_seq_layer_desc d;
    int src = 0;                       // layer whose SeqWeights it uses
    // derived
    int inner = 0, conv_ch = 0, dproj = 0;            // mamba2: heads*vdim, inner + 2*groups*state, 2*inner + 2*groups*state + heads
    int nq = 0, nk = 0, nv = 0, ng = 0, lproj = 0;    // attention projection widths
    int rn = 0;                                       // RWKV heads*dim
    int dproj_ld = 0, lproj_ld = 0;                   // row pitch of the projection outputs (multiples of 8: tensor-core epilogue)
};

struct SeqModel {
    b2_seq_model_desc d;
    std::vector<SeqLayerInfo> layers;
    std::vector<SeqWeights> w;
    DevBuf embed, head, final_w, final_b;
    std::map<std::string, int> got;
    int w_dtype = DT_BF16;             // dtype of the Linear weights and the embedding table on the device
    int rows = 0;                      // workspace rows
    // workspaces (fp32 unless noted)
    DevBuf x, proj, act, y, gated, mixout, mixes, rp, wl1, wlog, ff, xn, tok, want;
    DevBuf a16;                        // bf16 copy of a GEMM's A operand (tensor-core path of the bf16 compute mode)
    int a16_w = 0;
    DevBuf segs, row_slot, row_pos;
    int proj_w = 0, act_w = 0, y_w = 0, rp_w = 0, rank_w = 0, ff_w = 0;
};

struct SeqLayerState {
    DevBuf ssm, conv_tail;             // mamba2: [slots][heads][state][vdim], [slots][taps-1][channels]
    DevBuf kc, vc, bucket_of;          // attention: [slots][G][Smax][dk], [slots][G][Smax][dv], int32 [Smax]
    DevBuf wkv, prev;                  // RWKV: [slots][heads][dim][dim], [slots][width]
};
struct SeqState {
    std::vector<SeqLayerState> layer;
    DevBuf attn_partial;
    int nsplit_max = 1;
};

namespace {

const size_t F4 = sizeof(float);
size_t esz(int dt) { return dt == DT_F32 ? 4 : 2; }

int64_t numel(const int64_t* shape, int ndim) {
    int64_t n = 1;
    for (int i = 0; i < ndim; ++i) n *= shape[i];
    return n;
}

// host-or-device tensor of `dtype` -> device buffer of `to` (DT_F32 or DT_BF16), at element offset `off` of a buffer of
// `total` elements (allocated on first use)
int put_tensor(DevBuf& buf, int to, size_t total, size_t off, const void* src, int dtype, int64_t n) {
    if (buf.p == nullptr) {
        B2_TRY(buf.alloc(total * esz(to)));
        B2_CUDA_CHECK(cudaMemset(buf.p, 0, total * esz(to)));
    }
    cudaPointerAttributes attr;
    bool on_device = false;
    if (cudaPointerGetAttributes(&attr, src) == cudaSuccess) on_device = attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged;
    else cudaGetLastError();
    const size_t sz = dtype == DT_F32 ? 4 : 2;
    DevBuf tmp;
    const void* dsrc = src;
    if (!on_device) {
        B2_TRY(tmp.alloc((size_t)n * sz));
        B2_CUDA_CHECK(cudaMemcpy(tmp.p, src, (size_t)n * sz, cudaMemcpyDefault));
        dsrc = tmp.p;
    }
    int r = to == DT_F32 ? convert_to_f32(dsrc, dtype, buf.as<float>() + off, n, 0)
                         : convert_to_bf16(dsrc, dtype, buf.as<__nv_bfloat16>() + off, n, 0);
    cudaError_t e = cudaStreamSynchronize(0);
    tmp.free();
    if (r != 0) return r;
    B2_CUDA_CHECK(e);
    return 0;
}

int want_shape(const char* key, const int64_t* shape, int ndim, int64_t a, int64_t b = -1) {
    const bool ok = b < 0 ? (numel(shape, ndim) == a) : (ndim == 2 && shape[0] == a && shape[1] == b);
    if (!ok) {
        char got[96] = {0};
        int o = 0;
        for (int i = 0; i < ndim && o < 80; ++i) o += snprintf(got + o, sizeof(got) - o, "%s%lld", i ? "x" : "", (long long)shape[i]);
        if (b < 0) set_error("set_weight(%s): shape %s, expected %lld elements", key, got, (long long)a);
        else set_error("set_weight(%s): shape %s, expected %lldx%lld", key, got, (long long)a, (long long)b);
        return -1;
    }
    return 0;
}

bool tc_enabled() {  // B2_SEQ_TC=0: every Linear on the FMA kernels (A/B runs, tests of the two paths against each other)
    const char* e = getenv("B2_SEQ_TC");
    return !(e != nullptr && e[0] == '0');
}

int tc_min_rows() {  // fewest rows that take the tensor-core GEMM (below: the weight-streaming FMA kernels)
    const char* e = getenv("B2_SEQ_TC_MIN_ROWS");
    const int v = e != nullptr ? atoi(e) : 0;
    // measured at widths 2048 / 4096 (decode step, ms): 4 rows 0.76 / 1.38 on the tile GEMM vs 0.78 / 1.48 on the FMA kernel,
    // 8 rows 0.87 / 1.59 vs 1.14 / 3.45; 2 rows 0.71 / 1.28 vs 0.62 / 1.10
    return v >= 1 ? v : 4;
}

struct Lin {  // one Linear call on the model's compute dtype
    const b2_model* m;
    cudaStream_t st;
    int operator()(const float* A, int64_t lda, const DevBuf& W, int N, int K, float* out, int64_t ldo, int M, int act = LIN_NONE,
                   float alpha = 1.f, int accumulate = 0, const float* bias = nullptr, size_t w_row0 = 0) const {
        LinearArgs a;
        const SeqModel& s = *m->seq;
        a.A = A; a.lda = lda; a.ldw = K; a.w_dtype = s.w_dtype;
        a.W = reinterpret_cast<const char*>(W.p) + w_row0 * (size_t)K * esz(s.w_dtype);
        a.bias = bias; a.out = out; a.ld_out = ldo; a.M = M; a.N = N; a.K = K; a.act = act; a.alpha = alpha; a.accumulate = accumulate;
        a.round_a = s.d.compute == B2_COMPUTE_BF16;
        // bf16 compute, a portion of a prompt: the tcgen05 GEMM on a bf16 copy of A (weights are stored with their rows
        // padded to a multiple of 8, zero-filled, so N rounds up; the pitch of every projection buffer is a multiple of 8)
        const int Np = (N + 7) / 8 * 8;
        if (a.round_a && M >= tc_min_rows() && N >= 32 && K % 8 == 0 && K >= 32 && K <= s.a16_w && ldo % 8 == 0 && Np <= ldo && bias == nullptr &&
            w_row0 == 0 && tc_enabled()) {
            B2_TRY(cast_rows_bf16(A, lda, s.a16.p, K, M, K, st));
            GemmArgs g;
            g.A = s.a16.p; g.lda = K; g.W = W.p; g.ldw = K; g.out = out; g.ld_out = (int)ldo; g.out_fp32 = 1;
            g.M = M; g.N = Np; g.K = K; g.act = ACT_NONE; g.post = act; g.alpha = alpha; g.accumulate = accumulate;
            return gemm_bf16(g, st);
        }
        return linear_f32(a, st);
    }
};

int attn_nsplit(int rows, int G, int max_seq) {
    // a decode step has few (row, key/value head) CTAs: cut the keys so that the step fills the SMs twice over, but keep
    // at least 64 keys per cut at the cache's capacity
    if (rows > 8) return 1;
    int n = (2 * num_sms()) / (rows * G);
    const int cap = max_seq / 64;
    if (n > cap) n = cap;
    if (n > 64) n = 64;
    return n < 1 ? 1 : n;
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------------
// forward over R rows described by the model's row map (nseg segments). x holds the embedded rows on entry.
// ------------------------------------------------------------------------------------------------------------------
static int seq_forward(b2_model* m, b2_kv* kv, int R, int nseg, float* resid_out, cudaStream_t st) {
    SeqModel& s = *m->seq;
    SeqState& state = *kv->seq;
    const int width = s.d.width;
    const float eps = s.d.norm_eps;
    const Lin lin{m, st};
    float* x = s.x.as<float>();
    float* mix = s.mixout.as<float>();
    const SeqSeg* segs = s.segs.as<SeqSeg>();
    const int max_n = nseg == 1 ? R : 1;  // a prompt portion is one segment of R rows; a decode step is R segments of one row
    for (size_t li = 0; li < s.layers.size(); ++li) {
        const SeqLayerInfo& L = s.layers[li];
        const b2_seq_layer_desc& d = L.d;
        SeqWeights& W = s.w[L.src];
        SeqLayerState& S = state.layer[li];
        if (d.type == B2_MIXER_MAMBA2) {
            float* proj = s.proj.as<float>();
            const int gn = d.m_groups * d.m_state;
            B2_TRY(lin(x, width, W.in_w, L.dproj, width, proj, L.dproj_ld, R));
            float* act = s.act.as<float>();  // [R, conv_ch] = silu(conv(x | B | C))
            B2_TRY(causal_conv_silu_f32(proj + L.inner, L.dproj_ld, W.conv_w.as<float>(), W.conv_b.as<float>(), S.conv_tail.as<float>(), act,
                                        L.conv_ch, L.conv_ch, d.m_conv, segs, nseg, max_n, st));
            ScanArgs sa;
            sa.mode = SCAN_SSD;
            sa.v = act; sa.ldv = L.conv_ch;
            sa.k = act + L.inner; sa.ldk = L.conv_ch;
            sa.q = act + L.inner + gn; sa.ldq = L.conv_ch;
            sa.decay_in = proj + 2 * L.inner + 2 * gn; sa.ldd = L.dproj_ld;
            sa.dt_bias = W.dt_bias.as<float>(); sa.a_log = W.a_log.as<float>(); sa.skip = W.skip.as<float>();
            sa.state = S.ssm.as<float>();
            sa.y = s.y.as<float>(); sa.ldy = L.inner;
            sa.heads = d.m_heads; sa.groups = d.m_groups; sa.dk = d.m_state; sa.dv = d.m_vdim;
            sa.segs = segs; sa.nseg = nseg;
            B2_TRY(linear_scan_f32(sa, st));
            B2_TRY(gated_group_rmsnorm_f32(s.y.as<float>(), L.inner, proj, L.dproj_ld, W.mnorm.as<float>(), s.gated.as<float>(), L.inner, R, L.inner,
                                           L.inner / d.m_norm_groups, 1, eps, st));
            B2_TRY(lin(s.gated.as<float>(), L.inner, W.o_w, width, L.inner, mix, width, R));
        } else {
            // ---- left: attention -------------------------------------------------------------------------------------
            float* proj = s.proj.as<float>();  // [R, nq | nk | nv | ng]
            B2_TRY(lin(x, width, W.lproj_w, L.lproj, width, proj, L.lproj_ld, R));
            BiasAttnArgs aa;
            aa.q = proj; aa.ldq = L.lproj_ld;
            aa.k = proj + L.nq; aa.ldk = L.lproj_ld;
            aa.v = proj + L.nq + L.nk; aa.ldv = L.lproj_ld;
            aa.kcache = S.kc.as<float>(); aa.vcache = S.vc.as<float>();
            aa.out = s.y.as<float>(); aa.ldo = L.ng;
            aa.rel = W.rel.as<float>(); aa.bucket_of = S.bucket_of.as<int32_t>();
            aa.H = d.a_heads; aa.G = d.a_kv_heads; aa.dk = d.a_dim; aa.dv = d.a_vdim; aa.Smax = kv->max_seq; aa.rows = R;
            aa.eps = eps; aa.scale = d.a_scale; aa.softcap = d.a_softcap; aa.temp_coef = d.a_temp_coef; aa.temp_every = d.a_temp_every;
            aa.row_slot = s.row_slot.as<int32_t>(); aa.row_pos = s.row_pos.as<int32_t>();
            aa.nsplit = attn_nsplit(R, d.a_kv_heads, kv->max_seq);
            aa.tile_rows = max_n;
            if (aa.nsplit > state.nsplit_max) aa.nsplit = state.nsplit_max;
            aa.partial = state.attn_partial.as<float>();
            B2_TRY(attn_prepare_f32(aa, st));
            B2_TRY(attn_bias_f32(aa, st));
            B2_TRY(sigmoid_gate_f32(s.y.as<float>(), L.ng, proj + L.nq + L.nk + L.nv, L.lproj_ld, s.gated.as<float>(), L.ng, R, L.ng, st));
            B2_TRY(lin(s.gated.as<float>(), L.ng, W.lo_w, width, L.ng, mix, width, R, LIN_NONE, d.left_scale));
            // ---- right: RWKV time mixing -------------------------------------------------------------------------------
            const size_t ms = (size_t)s.rows * width;  // stride between the five mixes (r, k, v, g, w)
            float* mixes = s.mixes.as<float>();
            B2_TRY(token_shift_mix_f32(x, W.mu.as<float>(), S.prev.as<float>(), mixes, ms, width, 5, segs, nseg, max_n, st));
            float* rp = s.rp.as<float>();      // [4][rows][rn]: r, k, v, g
            const size_t rs = (size_t)s.rows * L.rn;
            B2_TRY(lin(mixes + 0 * ms, width, W.r_w, L.rn, width, rp + 0 * rs, L.rn, R));
            B2_TRY(lin(mixes + 1 * ms, width, W.k_w, L.rn, width, rp + 1 * rs, L.rn, R));
            B2_TRY(lin(mixes + 2 * ms, width, W.v_w, L.rn, width, rp + 2 * rs, L.rn, R));
            B2_TRY(lin(mixes + 3 * ms, width, W.g_w, L.rn, width, rp + 3 * rs, L.rn, R));
            B2_TRY(lin(mixes + 4 * ms, width, W.w1, d.r_decay_rank, width, s.wl1.as<float>(), d.r_decay_rank, R, LIN_TANH));
            B2_TRY(lin(s.wl1.as<float>(), d.r_decay_rank, W.w2, L.rn, d.r_decay_rank, s.wlog.as<float>(), L.rn, R, LIN_NONE, 1.f, 0, W.w0.as<float>()));
            ScanArgs sa;
            sa.mode = SCAN_RWKV;
            sa.q = rp; sa.ldq = L.rn;
            sa.k = rp + rs; sa.ldk = L.rn;
            sa.v = rp + 2 * rs; sa.ldv = L.rn;
            sa.decay_in = s.wlog.as<float>(); sa.ldd = L.rn;
            sa.bonus = W.bonus.as<float>();
            sa.state = S.wkv.as<float>();
            sa.y = s.y.as<float>(); sa.ldy = L.rn;
            sa.heads = d.r_heads; sa.groups = d.r_heads; sa.dk = d.r_dim; sa.dv = d.r_dim;
            sa.segs = segs; sa.nseg = nseg;
            B2_TRY(linear_scan_f32(sa, st));
            B2_TRY(gated_group_rmsnorm_f32(s.y.as<float>(), L.rn, rp + 3 * rs, L.rn, W.rnorm.as<float>(), s.gated.as<float>(), L.rn, R, L.rn, d.r_dim,
                                           0, eps, st));
            B2_TRY(lin(s.gated.as<float>(), L.rn, W.ro_w, width, L.rn, mix, width, R, LIN_NONE, d.right_scale, 1));
        }
        B2_TRY(layernorm_add_f32(x, mix, W.norm1.as<float>(), W.norm1_b.as<float>(), R, width, eps, st));
        if (d.ff > 0) {
            B2_TRY(lin(x, width, W.up_w, d.ff, width, s.ff.as<float>(), d.ff, R, LIN_RELU_SQ));
            B2_TRY(lin(s.ff.as<float>(), d.ff, W.down_w, width, d.ff, mix, width, R));
            B2_TRY(layernorm_add_f32(x, mix, W.norm2.as<float>(), W.norm2_b.as<float>(), R, width, eps, st));
        }
        if (resid_out != nullptr)
            B2_CUDA_CHECK(cudaMemcpyAsync(resid_out + li * (size_t)R * width, x, (size_t)R * width * F4, cudaMemcpyDeviceToDevice, st));
    }
    return 0;
}

// one decode step over the slots [slot0, slot0 + B): kv->tok -> logits (m->logits) -> token selection, lengths += 1
int seq_decode_launch(b2_model* m, b2_kv* kv, int B, int slot0, cudaStream_t st) {
    SeqModel& s = *m->seq;
    RowMap rm{s.segs.as<SeqSeg>(), s.row_slot.as<int32_t>(), s.row_pos.as<int32_t>()};
    B2_TRY(rowmap_decode(rm, kv->len_dev.as<int32_t>(), kv->sstate.as<SampleState>(), kv->rows_dev.as<RowState>(), slot0, B, st));
    B2_TRY(embed_rows_f32(kv->tok.as<int32_t>() + slot0, s.embed.p, s.w_dtype, s.x.as<float>(), B, s.d.width, s.d.vocab, m->err_dev, st));
    B2_TRY(seq_forward(m, kv, B, B, nullptr, st));
    B2_TRY(layernorm_gather_f32(s.x.as<float>(), nullptr, s.final_w.as<float>(), s.final_b.as<float>(), s.xn.as<float>(), B, s.d.width, s.d.norm_eps, st));
    const Lin lin{m, st};
    B2_TRY(lin(s.xn.as<float>(), s.d.width, s.head, s.d.vocab, s.d.width, m->logits.as<float>(), s.d.vocab, B));
    B2_TRY(sample_publish(m->logits.as<float>(), s.d.vocab, B, kv->sstate.as<SampleState>(), kv->rows_dev.as<RowState>() + slot0,
                          kv->tok.as<int32_t>() + slot0, kv->out_tokens.as<int32_t>(), kv->step_counter.as<int32_t>(),
                          kv->len_dev.as<int32_t>() + slot0, kv->ring_dev, kv->ring_cap, SP_SELECT | SP_WRITE_OUT | SP_BUMP, 0, st));
    return 0;
}

// ------------------------------------------------------------------------------------------------------------------
// weights
// ------------------------------------------------------------------------------------------------------------------
int seq_set_weight(b2_model* m, const char* key, const void* ptr, const int64_t* shape, int ndim, int dt) {
    SeqModel& s = *m->seq;
    const int width = s.d.width, V = s.d.vocab, WD = s.w_dtype;
    const std::string k(key);
    if (k == "embed") { B2_TRY(want_shape(key, shape, ndim, V, width)); s.got[k] = 1; return put_tensor(s.embed, WD, (size_t)V * width, 0, ptr, dt, (int64_t)V * width); }
    if (k == "head") { B2_TRY(want_shape(key, shape, ndim, V, width)); s.got[k] = 1; return put_tensor(s.head, WD, (size_t)((V + 7) / 8 * 8) * width, 0, ptr, dt, (int64_t)V * width); }
    if (k == "final.norm") { B2_TRY(want_shape(key, shape, ndim, width)); s.got[k] = 1; return put_tensor(s.final_w, DT_F32, width, 0, ptr, dt, width); }
    if (k == "final.norm.b") { B2_TRY(want_shape(key, shape, ndim, width)); s.got[k] = 1; return put_tensor(s.final_b, DT_F32, width, 0, ptr, dt, width); }
    int li = -1, used = 0;
    if (sscanf(key, "l%d.%n", &li, &used) != 1 || used == 0 || li < 0 || li >= (int)s.layers.size()) {
        set_error("set_weight: unknown tensor '%s'", key);
        return -1;
    }
    const SeqLayerInfo& L = s.layers[li];
    B2_CHECK_ARG(L.src == li, "set_weight(%s): layer %d uses the tensors of layer %d and has none of its own", key, li, L.src);
    const b2_seq_layer_desc& d = L.d;
    SeqWeights& W = s.w[li];
    const std::string r = k.substr(used);
    auto vec = [&](DevBuf& b, int64_t n) -> int { B2_TRY(want_shape(key, shape, ndim, n)); W.got[r] = 1; return put_tensor(b, DT_F32, n, 0, ptr, dt, n); };
    // Linear weights are allocated with their rows padded to a multiple of 8 (zeros): the tensor-core GEMM wants N % 8 == 0
    auto mat = [&](DevBuf& b, int64_t o, int64_t i) -> int { B2_TRY(want_shape(key, shape, ndim, o, i)); W.got[r] = 1; return put_tensor(b, WD, (size_t)((o + 7) / 8 * 8) * i, 0, ptr, dt, o * i); };
    if (r == "norm1") return vec(W.norm1, width);
    if (r == "norm1.b") return vec(W.norm1_b, width);
    if (d.ff > 0) {
        if (r == "norm2") return vec(W.norm2, width);
        if (r == "norm2.b") return vec(W.norm2_b, width);
        if (r == "mlp.up") return mat(W.up_w, d.ff, width);
        if (r == "mlp.down") return mat(W.down_w, width, d.ff);
    }
    if (d.type == B2_MIXER_MAMBA2) {
        if (r == "mix.in") return mat(W.in_w, L.dproj, width);
        if (r == "mix.conv") { B2_TRY(want_shape(key, shape, ndim, L.conv_ch, d.m_conv)); W.got[r] = 1; return put_tensor(W.conv_w, DT_F32, (size_t)L.conv_ch * d.m_conv, 0, ptr, dt, (int64_t)L.conv_ch * d.m_conv); }
        if (r == "mix.conv.b") return vec(W.conv_b, L.conv_ch);
        if (r == "mix.dt_bias") return vec(W.dt_bias, d.m_heads);
        if (r == "mix.A_log") return vec(W.a_log, d.m_heads);
        if (r == "mix.D") return vec(W.skip, d.m_heads);
        if (r == "mix.norm") return vec(W.mnorm, L.inner);
        if (r == "mix.o") return mat(W.o_w, width, L.inner);
    } else {
        // the four attention projections share their input: one [nq + nk + nv + ng, width] matrix, one product
        const char* parts[4] = {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g"};
        const int sizes[4] = {L.nq, L.nk, L.nv, L.ng};
        size_t row0 = 0;
        for (int j = 0; j < 4; ++j) {
            if (r == parts[j]) {
                B2_TRY(want_shape(key, shape, ndim, sizes[j], width));
                W.got[r] = 1;
                return put_tensor(W.lproj_w, WD, (size_t)L.lproj_ld * width, row0 * width, ptr, dt, (int64_t)sizes[j] * width);
            }
            row0 += sizes[j];
        }
        if (r == "mix.left.rel") { B2_TRY(want_shape(key, shape, ndim, d.a_rel_rows, d.a_heads)); W.got[r] = 1; return put_tensor(W.rel, DT_F32, (size_t)d.a_rel_rows * d.a_heads, 0, ptr, dt, (int64_t)d.a_rel_rows * d.a_heads); }
        if (r == "mix.left.o") return mat(W.lo_w, width, L.ng);
        const char* mus[5] = {"mix.right.mu.r", "mix.right.mu.k", "mix.right.mu.v", "mix.right.mu.g", "mix.right.mu.w"};
        for (int j = 0; j < 5; ++j)
            if (r == mus[j]) {
                B2_TRY(want_shape(key, shape, ndim, width));
                W.got[r] = 1;
                return put_tensor(W.mu, DT_F32, (size_t)5 * width, (size_t)j * width, ptr, dt, width);
            }
        if (r == "mix.right.r") return mat(W.r_w, L.rn, width);
        if (r == "mix.right.k") return mat(W.k_w, L.rn, width);
        if (r == "mix.right.v") return mat(W.v_w, L.rn, width);
        if (r == "mix.right.g") return mat(W.g_w, L.rn, width);
        if (r == "mix.right.w1") return mat(W.w1, d.r_decay_rank, width);
        if (r == "mix.right.w2") return mat(W.w2, L.rn, d.r_decay_rank);
        if (r == "mix.right.w0") return vec(W.w0, L.rn);
        if (r == "mix.right.u") return vec(W.bonus, L.rn);
        if (r == "mix.right.norm") return vec(W.rnorm, L.rn);
        if (r == "mix.right.o") return mat(W.ro_w, width, L.rn);
    }
    set_error("set_weight: tensor '%s' does not belong to a layer of this kind", key);
    return -1;
}

static std::vector<std::string> required_of(const SeqLayerInfo& L) {
    std::vector<std::string> v = {"norm1", "norm1.b"};
    if (L.d.ff > 0) for (const char* n : {"norm2", "norm2.b", "mlp.up", "mlp.down"}) v.push_back(n);
    if (L.d.type == B2_MIXER_MAMBA2) {
        for (const char* n : {"mix.in", "mix.conv", "mix.conv.b", "mix.dt_bias", "mix.A_log", "mix.D", "mix.norm", "mix.o"}) v.push_back(n);
    } else {
        for (const char* n : {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.g", "mix.left.rel", "mix.left.o", "mix.right.mu.r", "mix.right.mu.k",
                              "mix.right.mu.v", "mix.right.mu.g", "mix.right.mu.w", "mix.right.r", "mix.right.k", "mix.right.v", "mix.right.g",
                              "mix.right.w1", "mix.right.w2", "mix.right.w0", "mix.right.u", "mix.right.norm", "mix.right.o"})
            v.push_back(n);
    }
    return v;
}

int seq_finalize(b2_model* m) {
    SeqModel& s = *m->seq;
    std::string missing;
    for (const char* n : {"embed", "head", "final.norm", "final.norm.b"})
        if (!s.got.count(n) && missing.size() < 600) { missing += n; missing += ' '; }
    for (size_t i = 0; i < s.layers.size(); ++i) {
        if (s.layers[i].src != (int)i) continue;
        for (const std::string& n : required_of(s.layers[i]))
            if (!s.w[i].got.count(n) && missing.size() < 600) missing += "l" + std::to_string(i) + "." + n + " ";
    }
    if (!missing.empty()) {
        set_error("b2_model_finalize: missing tensors: %s", missing.c_str());
        return -3;
    }
    const int width = s.d.width;
    int pw = 1, aw = 1, yw = 1, rw = 1, kw = 1, fw = 1;
    for (const SeqLayerInfo& L : s.layers) {
        if (L.d.type == B2_MIXER_MAMBA2) {
            pw = std::max(pw, L.dproj_ld); aw = std::max(aw, L.conv_ch); yw = std::max(yw, L.inner);
        } else {
            pw = std::max(pw, L.lproj_ld); yw = std::max(yw, std::max(L.ng, L.rn)); rw = std::max(rw, L.rn); kw = std::max(kw, L.d.r_decay_rank);
        }
        fw = std::max(fw, L.d.ff);
    }
    s.proj_w = pw; s.act_w = aw; s.y_w = yw; s.rp_w = rw; s.rank_w = kw; s.ff_w = fw;
    const size_t R = (size_t)s.rows;
    B2_TRY(s.x.alloc(R * width * F4));
    B2_TRY(s.proj.alloc(R * pw * F4));
    B2_TRY(s.act.alloc(R * aw * F4));
    B2_TRY(s.y.alloc(R * yw * F4));
    B2_TRY(s.gated.alloc(R * yw * F4));
    B2_TRY(s.mixout.alloc(R * width * F4));
    B2_TRY(s.mixes.alloc(5 * R * width * F4));
    B2_TRY(s.rp.alloc(4 * R * rw * F4));
    B2_TRY(s.wl1.alloc(R * kw * F4));
    B2_TRY(s.wlog.alloc(R * rw * F4));
    B2_TRY(s.ff.alloc(R * fw * F4));
    B2_TRY(s.xn.alloc(R * width * F4));
    {
        int kmax = width;
        for (const SeqLayerInfo& L : s.layers) kmax = std::max(kmax, std::max(std::max(L.inner, L.ng), std::max(L.rn, L.d.ff)));
        s.a16_w = (kmax + 7) / 8 * 8;
        if (s.d.compute == B2_COMPUTE_BF16) B2_TRY(s.a16.alloc(R * s.a16_w * 2));
    }
    B2_TRY(s.tok.alloc(R * 4));
    B2_TRY(s.want.alloc(R * 4));
    B2_TRY(s.segs.alloc((size_t)std::max(1, s.d.max_batch) * sizeof(SeqSeg)));
    B2_TRY(s.row_slot.alloc(R * 4));
    B2_TRY(s.row_pos.alloc(R * 4));
    B2_TRY(m->logits.alloc((size_t)s.d.max_batch * s.d.vocab * 4));
    return 0;
}

void seq_model_free(b2_model* m) {
    if (m->seq == nullptr) return;
    SeqModel& s = *m->seq;
    for (SeqWeights& W : s.w) {
        DevBuf* bs[] = {&W.norm1, &W.norm1_b, &W.norm2, &W.norm2_b, &W.in_w, &W.conv_w, &W.conv_b, &W.dt_bias, &W.a_log, &W.skip, &W.mnorm, &W.o_w,
                        &W.lproj_w, &W.rel, &W.lo_w, &W.mu, &W.r_w, &W.k_w, &W.v_w, &W.g_w, &W.w1, &W.w2, &W.w0, &W.bonus, &W.rnorm, &W.ro_w,
                        &W.up_w, &W.down_w};
        for (DevBuf* b : bs) b->free();
    }
    DevBuf* bs[] = {&s.embed, &s.head, &s.final_w, &s.final_b, &s.x, &s.proj, &s.act, &s.y, &s.gated, &s.mixout, &s.mixes, &s.rp, &s.wl1, &s.wlog,
                    &s.ff, &s.xn, &s.tok, &s.want, &s.segs, &s.row_slot, &s.row_pos, &s.a16};
    for (DevBuf* b : bs) b->free();
    delete m->seq;
    m->seq = nullptr;
}

// ------------------------------------------------------------------------------------------------------------------
// per-cache state
// ------------------------------------------------------------------------------------------------------------------
static int distance_bucket(int n, int rows, double far_) {
    const int half = rows / 2;
    if (n < half || half == 0) return n < rows ? n : rows - 1;
    const double v = log((double)n / half) / log(far_ / half) * (rows - half);
    const long b = half + (long)floor(v);
    return (int)(b < rows - 1 ? b : rows - 1);
}

int64_t seq_kv_bytes(const b2_model* m, int B, int Smax) {
    int64_t n = 0;
    for (const SeqLayerInfo& L : m->seq->layers) {
        const b2_seq_layer_desc& d = L.d;
        if (d.type == B2_MIXER_MAMBA2) n += (int64_t)B * d.m_heads * d.m_state * d.m_vdim + (int64_t)B * (d.m_conv - 1) * L.conv_ch;
        else n += (int64_t)B * d.a_kv_heads * Smax * (d.a_dim + d.a_vdim) + (int64_t)B * d.r_heads * d.r_dim * d.r_dim + (int64_t)B * m->seq->d.width;
    }
    return n * 4;
}

int seq_kv_alloc(b2_kv* kv) {
    const b2_model* m = kv->m;
    const SeqModel& s = *m->seq;
    const size_t B = kv->max_batch, Smax = kv->max_seq;
    kv->seq = new SeqState();
    kv->seq->layer.resize(s.layers.size());
    int maxH = 1, maxdv = 1;
    for (size_t li = 0; li < s.layers.size(); ++li) {
        const SeqLayerInfo& L = s.layers[li];
        const b2_seq_layer_desc& d = L.d;
        SeqLayerState& S = kv->seq->layer[li];
        if (d.type == B2_MIXER_MAMBA2) {
            B2_TRY(S.ssm.alloc(B * d.m_heads * d.m_state * d.m_vdim * F4));
            B2_TRY(S.conv_tail.alloc(std::max<size_t>(1, B * (d.m_conv - 1) * L.conv_ch) * F4));
            cudaMemset(S.ssm.p, 0, S.ssm.bytes);
            cudaMemset(S.conv_tail.p, 0, S.conv_tail.bytes);
        } else {
            B2_TRY(S.kc.alloc(B * d.a_kv_heads * Smax * d.a_dim * F4));
            B2_TRY(S.vc.alloc(B * d.a_kv_heads * Smax * d.a_vdim * F4));
            B2_TRY(S.wkv.alloc(B * d.r_heads * d.r_dim * d.r_dim * F4));
            B2_TRY(S.prev.alloc(B * s.d.width * F4));
            B2_TRY(S.bucket_of.alloc(Smax * 4));
            cudaMemset(S.kc.p, 0, S.kc.bytes);
            cudaMemset(S.vc.p, 0, S.vc.bytes);
            cudaMemset(S.wkv.p, 0, S.wkv.bytes);
            cudaMemset(S.prev.p, 0, S.prev.bytes);
            std::vector<int32_t> tab(Smax);
            for (size_t n = 0; n < Smax; ++n) tab[n] = distance_bucket((int)n, d.a_rel_rows, (double)d.a_bias_max);
            B2_CUDA_CHECK(cudaMemcpy(S.bucket_of.p, tab.data(), Smax * 4, cudaMemcpyHostToDevice));
            maxH = std::max(maxH, d.a_heads);
            maxdv = std::max(maxdv, d.a_vdim);
        }
    }
    kv->seq->nsplit_max = 64;
    B2_TRY(kv->seq->attn_partial.alloc((size_t)8 * maxH * kv->seq->nsplit_max * (maxdv + 2) * F4));
    return 0;
}

void seq_kv_free(b2_kv* kv) {
    if (kv->seq == nullptr) return;
    for (SeqLayerState& S : kv->seq->layer) {
        DevBuf* bs[] = {&S.ssm, &S.conv_tail, &S.kc, &S.vc, &S.bucket_of, &S.wkv, &S.prev};
        for (DevBuf* b : bs) b->free();
    }
    kv->seq->attn_partial.free();
    delete kv->seq;
    kv->seq = nullptr;
}

}  // namespace b2

using namespace b2;

// ==================================================================================================================
// C ABI
// ==================================================================================================================
extern "C" {

int b2_seq_model_create(const b2_seq_model_desc* desc, const b2_seq_layer_desc* layers, b2_model** out) {
    B2_CHECK_ARG(desc && layers && out, "b2_seq_model_create: null argument");
    const b2_seq_model_desc& d = *desc;
    B2_CHECK_ARG(d.width > 0 && d.vocab > 0 && d.n_layers > 0, "b2_seq_model_create: width %d, vocab %d, %d layers", d.width, d.vocab, d.n_layers);
    B2_CHECK_ARG(d.compute == B2_COMPUTE_BF16 || d.compute == B2_COMPUTE_F32, "b2_seq_model_create: unknown compute mode %d", d.compute);
    B2_CHECK_ARG(d.max_batch >= 1 && d.max_rows >= 1, "b2_seq_model_create: bad workspace sizing");
    B2_CHECK_ARG(d.norm_eps >= 0.f, "b2_seq_model_create: negative eps");
    SeqModel* s = new SeqModel();
    s->d = d;
    s->w_dtype = d.compute == B2_COMPUTE_F32 ? DT_F32 : DT_BF16;
    s->rows = std::max(d.max_batch, d.max_rows);
    s->layers.resize(d.n_layers);
    s->w.resize(d.n_layers);
    // a layer may name ANY other layer as the owner of its tensors (an owner that itself borrows is followed to its owner)
    for (int i = 0; i < d.n_layers; ++i) s->layers[i].d = layers[i];
    for (int i = 0; i < d.n_layers; ++i) {
        int j = i, hops = 0;
        while (j >= 0 && j < d.n_layers && s->layers[j].d.weights_of >= 0 && s->layers[j].d.weights_of != j && hops <= d.n_layers) {
            j = s->layers[j].d.weights_of;
            ++hops;
        }
        if (j < 0 || j >= d.n_layers || hops > d.n_layers) {
            set_error("b2_seq_model_create: layer %d: weights_of does not lead to a layer that owns its tensors", i);
            delete s;
            return -1;
        }
        s->layers[i].src = j;
    }
    for (int i = 0; i < d.n_layers; ++i) {
        SeqLayerInfo& L = s->layers[i];
        const b2_seq_layer_desc& l = L.d;
        const char* why = nullptr;
        if (l.ff < 0) why = "negative feed-forward width";
        else if (l.type == B2_MIXER_MAMBA2) {
            if (l.m_heads < 1 || l.m_vdim < 1 || l.m_state < 1 || l.m_groups < 1 || l.m_heads % l.m_groups) why = "mamba2: heads must be a positive multiple of groups";
            else if (l.m_conv < 1 || l.m_conv > 16) why = "mamba2: 1..16 convolution taps";
            else if (l.m_norm_groups < 1 || (l.m_heads * l.m_vdim) % l.m_norm_groups) why = "mamba2: norm_groups must divide heads*vdim";
            else if (l.m_state > 256) why = "mamba2: state size above 256";
            L.inner = l.m_heads * l.m_vdim;
            L.conv_ch = L.inner + 2 * l.m_groups * l.m_state;
            L.dproj = 2 * L.inner + 2 * l.m_groups * l.m_state + l.m_heads;
            L.dproj_ld = (L.dproj + 7) / 8 * 8;
        } else if (l.type == B2_MIXER_PARALLEL) {
            if (l.a_heads < 1 || l.a_kv_heads < 1 || l.a_heads % l.a_kv_heads) why = "attention: heads must be a positive multiple of kv_heads";
            else if (l.a_dim < 1 || l.a_dim > 256 || l.a_vdim < 1 || l.a_vdim > 256) why = "attention: head sizes 1..256";
            else if (l.a_rel_rows < 1 || !(l.a_bias_max > 0.f)) why = "attention: the distance bias needs rows and a positive far limit";
            else if (!(l.a_temp_every > 0.f)) why = "attention: q_temp.every must be positive";
            else if (l.r_heads < 1 || l.r_dim < 1 || l.r_dim > 256 || l.r_decay_rank < 1) why = "rwkv: heads, dim 1..256, decay rank";
            L.nq = l.a_heads * l.a_dim; L.nk = l.a_kv_heads * l.a_dim; L.nv = l.a_kv_heads * l.a_vdim; L.ng = l.a_heads * l.a_vdim;
            L.lproj = L.nq + L.nk + L.nv + L.ng;
            L.lproj_ld = (L.lproj + 7) / 8 * 8;
            L.rn = l.r_heads * l.r_dim;
        } else {
            why = "unknown mixer type";
        }
        if (why == nullptr && L.src != i) {
            b2_seq_layer_desc a = l, b = s->layers[L.src].d;
            a.weights_of = b.weights_of = -1;
            if (memcmp(&a, &b, sizeof(a)) != 0) why = "a layer that borrows weights must have the sizes of their owner";
        }
        if (why != nullptr) {
            set_error("b2_seq_model_create: layer %d: %s", i, why);
            delete s;
            return -1;
        }
    }
    b2_model* m = new b2_model();
    memset(&m->d, 0, sizeof(m->d));
    m->d.vocab = d.vocab; m->d.max_batch = d.max_batch; m->d.max_seq = d.max_rows; m->d.layers = d.n_layers; m->d.hidden = d.width;
    m->arch = B2_ARCH_LAYER_LIST;
    m->seq = s;
    cudaGetDevice(&m->device);
    *out = m;
    return 0;
}

int b2_append_tokens(b2_model* m, b2_kv* kv, int slot, const int32_t* tokens_host, int n, int restart, const int32_t* want_host, int n_want,
                     float* logits_out, float* resid_out, void* stream) {
    B2_CHECK_ARG(m && kv && kv->m == m && tokens_host, "b2_append_tokens: bad handle");
    B2_CHECK_ARG(m->arch == B2_ARCH_LAYER_LIST && m->finalized, "b2_append_tokens: needs a finalized layer-list model");
    SeqModel& s = *m->seq;
    B2_CHECK_ARG(slot >= 0 && slot < kv->max_batch, "b2_append_tokens: slot %d outside the cache (%d slots)", slot, kv->max_batch);
    B2_CHECK_ARG(n >= 1 && n <= s.d.max_rows, "b2_append_tokens: %d tokens in one call (at most %d)", n, s.d.max_rows);
    B2_CHECK_ARG(n_want >= 0 && n_want <= n && (n_want == 0 || (want_host && logits_out)), "b2_append_tokens: bad logits request");
    std::lock_guard<std::mutex> lk(m->mu);
    DeviceGuard dg(m->device);
    const int start = restart ? 0 : kv->len_host[slot];
    B2_CHECK_ARG(start + n <= kv->max_seq, "b2_append_tokens: %d + %d tokens exceed the cache's %d per slot", start, n, kv->max_seq);
    for (int i = 0; i < n_want; ++i) B2_CHECK_ARG(want_host[i] >= 0 && want_host[i] < n, "b2_append_tokens: wanted index %d outside the %d tokens", want_host[i], n);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    B2_TRY(ws_enter(m, st));
    B2_CUDA_CHECK(cudaMemcpyAsync(s.tok.p, tokens_host, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    RowMap rm{s.segs.as<SeqSeg>(), s.row_slot.as<int32_t>(), s.row_pos.as<int32_t>()};
    // a slot that starts over begins from position 0 whatever its device-side length says
    B2_TRY(rowmap_portion(rm, kv->len_dev.as<int32_t>(), slot, n, start == 0 ? 1 : 0, st));
    B2_TRY(embed_rows_f32(s.tok.as<int32_t>(), s.embed.p, s.w_dtype, s.x.as<float>(), n, s.d.width, s.d.vocab, m->err_dev, st));
    B2_TRY(seq_forward(m, kv, n, 1, resid_out, st));
    if (n_want > 0) {
        B2_CUDA_CHECK(cudaMemcpyAsync(s.want.p, want_host, (size_t)n_want * 4, cudaMemcpyHostToDevice, st));
        B2_TRY(layernorm_gather_f32(s.x.as<float>(), s.want.as<int32_t>(), s.final_w.as<float>(), s.final_b.as<float>(), s.xn.as<float>(), n_want,
                                    s.d.width, s.d.norm_eps, st));
        const Lin lin{m, st};
        cudaPointerAttributes attr;
        bool dev_out = cudaPointerGetAttributes(&attr, logits_out) == cudaSuccess && (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
        cudaGetLastError();
        if (dev_out) {
            B2_TRY(lin(s.xn.as<float>(), s.d.width, s.head, s.d.vocab, s.d.width, logits_out, s.d.vocab, n_want));
        } else {
            // host destination: through the projection workspace, in pieces of what it holds
            const int per = (int)std::max<size_t>(1, ((size_t)s.rows * s.proj_w) / s.d.vocab);
            for (int i0 = 0; i0 < n_want; i0 += per) {
                const int c = std::min(per, n_want - i0);
                B2_TRY(lin(s.xn.as<float>() + (size_t)i0 * s.d.width, s.d.width, s.head, s.d.vocab, s.d.width, s.proj.as<float>(), s.d.vocab, c));
                B2_CUDA_CHECK(cudaMemcpyAsync(logits_out + (size_t)i0 * s.d.vocab, s.proj.p, (size_t)c * s.d.vocab * 4, cudaMemcpyDeviceToHost, st));
                B2_CUDA_CHECK(cudaStreamSynchronize(st));
            }
        }
    }
    kv->len_host[slot] = start + n;
    return ws_leave(m, st);
}

int b2_kv_free_slot(b2_kv* kv, int slot, void* stream) {
    B2_CHECK_ARG(kv && slot >= 0 && slot < kv->max_batch, "b2_kv_free_slot: bad slot");
    std::lock_guard<std::mutex> lk(kv->m->mu);
    DeviceGuard dg(kv->m->device);
    B2_CUDA_CHECK(cudaMemsetAsync(kv->len_dev.as<int32_t>() + slot, 0, 4, reinterpret_cast<cudaStream_t>(stream)));
    kv->len_host[slot] = 0;
    return 0;
}

int64_t b2_kv_bytes(b2_model* m, int max_batch, int max_seq) {
    if (m == nullptr || max_batch < 1 || max_seq < 1) return -1;
    if (m->arch == B2_ARCH_LAYER_LIST) return seq_kv_bytes(m, max_batch, max_seq);
    return (int64_t)2 * m->d.layers * max_batch * m->d.heads * max_seq * m->hd * 2;
}

}  // extern "C"
