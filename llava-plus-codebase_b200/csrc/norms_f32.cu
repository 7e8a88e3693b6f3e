// fp32 normalisations and row helpers of the layer-list decoders: LayerNorm of a sublayer's output added to the residual
// stream, gathered LayerNorm in front of the output head, grouped unit-RMS norm with a SiLU gate (before or after the
// norm), embedding rows as fp32, the row map of a call. Statistics, sums and outputs are fp32 throughout; any width.
#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// sum over the block; every thread gets the result. `red` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();  // red may still be read from the previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
}

// mean, then the mean of squared deviations (two passes over the row, which sits in L1 after the first)
__device__ __forceinline__ void row_stats(const float* y, int cols, float eps, float* red, float& mean, float& rstd) {
    float s = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) s += y[c];
    mean = block_sum(s, red) / (float)cols;
    float q = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) { const float d = y[c] - mean; q = fmaf(d, d, q); }
    const float var = block_sum(q, red) / (float)cols;
    rstd = 1.f / sqrtf(var + eps);
}

__global__ void layernorm_add_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* yr = y + r * cols;
    float mean, rstd;
    row_stats(yr, cols, eps, red, mean, rstd);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) x[r * cols + c] += (yr[c] - mean) * rstd * gamma[c] + beta[c];
}

__global__ void layernorm_gather_kernel(const float* __restrict__ x, const int32_t* __restrict__ row_index, const float* __restrict__ gamma,
                                        const float* __restrict__ beta, float* __restrict__ out, int cols, float eps) {
    __shared__ float red[33];
    const size_t r = blockIdx.x;
    const float* xr = x + (size_t)(row_index != nullptr ? row_index[r] : (int)r) * cols;  // null index: row r itself
    float mean, rstd;
    row_stats(xr, cols, eps, red, mean, rstd);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[r * cols + c] = (xr[c] - mean) * rstd * gamma[c] + beta[c];
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// one warp per (row, group)
__global__ void gated_group_rmsnorm_kernel(const float* __restrict__ y, int64_t ldy, const float* __restrict__ z, int64_t ldz,
                                           const float* __restrict__ gamma, float* __restrict__ out, int64_t ldo, int rows, int groups, int group,
                                           int gate_first, float eps) {
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= rows * groups) return;
    const int r = w / groups, g = w % groups;
    const float* yr = y + (size_t)r * ldy + (size_t)g * group;
    const float* zr = z + (size_t)r * ldz + (size_t)g * group;
    float q = 0.f;
    for (int c = lane; c < group; c += 32) {
        const float v = gate_first ? yr[c] * silu_f(zr[c]) : yr[c];
        q = fmaf(v, v, q);
    }
    q = warp_sum(q);
    const float rinv = 1.f / sqrtf(q / (float)group + eps);
    float* o = out + (size_t)r * ldo + (size_t)g * group;
    for (int c = lane; c < group; c += 32) {
        const float gz = silu_f(zr[c]);
        o[c] = gate_first ? (yr[c] * gz) * rinv * gamma[g * group + c] : yr[c] * rinv * gamma[g * group + c] * gz;
    }
}

template <typename TT>
__global__ void embed_rows_kernel(const int32_t* __restrict__ tokens, const TT* __restrict__ table, float* __restrict__ x, int cols, int vocab,
                                  int* err_flag) {
    const size_t r = blockIdx.x;
    const int t = tokens[r];
    const bool ok = t >= 0 && t < vocab;
    if (!ok && threadIdx.x == 0 && err_flag != nullptr) err_flag[0] = 1;  // slot 0 = B2_ERR_TOKEN_RANGE
    for (int c = threadIdx.x; c < cols; c += blockDim.x) x[r * cols + c] = ok ? (float)table[(size_t)t * cols + c] : 0.f;
}

__global__ void sigmoid_gate_kernel(const float* __restrict__ a, int64_t lda, const float* __restrict__ g, int64_t ldg, float* __restrict__ out,
                                    int64_t ldo, int cols) {
    const size_t r = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c < cols) out[r * ldo + c] = a[r * lda + c] / (1.f + expf(-g[r * ldg + c]));
}

__global__ void rowmap_portion_kernel(SeqSeg* segs, int32_t* row_slot, int32_t* row_pos, int32_t* len, int slot, int n, int restart) {
    const int pos0 = restart ? 0 : len[slot];
    __syncthreads();
    for (int r = threadIdx.x; r < n; r += blockDim.x) { row_slot[r] = slot; row_pos[r] = pos0 + r; }
    if (threadIdx.x == 0) {
        segs[0].slot = slot; segs[0].row0 = 0; segs[0].n = n; segs[0].pos0 = pos0;
        len[slot] = pos0 + n;
    }
}

__global__ void rowmap_decode_kernel(SeqSeg* segs, int32_t* row_slot, int32_t* row_pos, const int32_t* len, const SampleState* sstate,
                                     const RowState* rows_state, int slot0, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const int slot = slot0 + b;
    // per-slot mode (continuous batching): a slot that is not armed keeps its state, cache rows and length
    const bool live = sstate == nullptr || rows_state == nullptr || sstate->per_row == 0 || rows_state[slot].active != 0;
    const int pos = len[slot];
    segs[b].slot = slot; segs[b].row0 = b; segs[b].n = live ? 1 : 0; segs[b].pos0 = pos;
    row_slot[b] = slot;
    row_pos[b] = live ? pos : -1;
}
}  // namespace

int layernorm_add_f32(float* x, const float* y, const float* gamma, const float* beta, int rows, int cols, float eps, cudaStream_t st) {
    B2_CHECK_ARG(x && y && gamma && beta && rows > 0 && cols > 0, "layernorm_add: bad argument");
    layernorm_add_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(x, y, gamma, beta, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int layernorm_gather_f32(const float* x, const int32_t* row_index, const float* gamma, const float* beta, float* out, int rows, int cols,
                         float eps, cudaStream_t st) {
    B2_CHECK_ARG(x && gamma && beta && out && rows > 0 && cols > 0, "layernorm_gather: bad argument");
    layernorm_gather_kernel<<<rows, cols >= 1024 ? 256 : 128, 0, st>>>(x, row_index, gamma, beta, out, cols, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int gated_group_rmsnorm_f32(const float* y, int64_t ldy, const float* z, int64_t ldz, const float* gamma, float* out, int64_t ldo, int rows,
                            int cols, int group, int gate_first, float eps, cudaStream_t st) {
    B2_CHECK_ARG(y && z && gamma && out && rows > 0 && group > 0 && cols % group == 0, "gated_group_rmsnorm: cols %d is not a multiple of the group %d",
                 cols, group);
    const int groups = cols / group, warps = rows * groups;
    gated_group_rmsnorm_kernel<<<(warps + 7) / 8, 256, 0, st>>>(y, ldy, z, ldz, gamma, out, ldo, rows, groups, group, gate_first, eps);
    B2_LAUNCH_CHECK();
    return 0;
}

int embed_rows_f32(const int32_t* tokens, const void* table, int table_dtype, float* x, int rows, int cols, int vocab, int* err_flag,
                   cudaStream_t st) {
    B2_CHECK_ARG(tokens && table && x && rows > 0, "embed_rows: bad argument");
    if (table_dtype == DT_F32)
        embed_rows_kernel<float><<<rows, 128, 0, st>>>(tokens, reinterpret_cast<const float*>(table), x, cols, vocab, err_flag);
    else
        embed_rows_kernel<__nv_bfloat16><<<rows, 128, 0, st>>>(tokens, reinterpret_cast<const __nv_bfloat16*>(table), x, cols, vocab, err_flag);
    B2_LAUNCH_CHECK();
    return 0;
}

int sigmoid_gate_f32(const float* a, int64_t lda, const float* g, int64_t ldg, float* out, int64_t ldo, int rows, int cols, cudaStream_t st) {
    B2_CHECK_ARG(a && g && out && rows > 0 && cols > 0, "sigmoid_gate: bad argument");
    sigmoid_gate_kernel<<<dim3((cols + 255) / 256, rows), 256, 0, st>>>(a, lda, g, ldg, out, ldo, cols);
    B2_LAUNCH_CHECK();
    return 0;
}

int rowmap_portion(const RowMap& rm, int32_t* len, int slot, int n, int restart, cudaStream_t st) {
    B2_CHECK_ARG(rm.segs && rm.row_slot && rm.row_pos && len && n > 0, "rowmap_portion: bad argument");
    rowmap_portion_kernel<<<1, 256, 0, st>>>(rm.segs, rm.row_slot, rm.row_pos, len, slot, n, restart);
    B2_LAUNCH_CHECK();
    return 0;
}

int rowmap_decode(const RowMap& rm, const int32_t* len, const SampleState* sstate, const RowState* rows_state, int slot0, int B, cudaStream_t st) {
    B2_CHECK_ARG(rm.segs && rm.row_slot && rm.row_pos && len && B > 0, "rowmap_decode: bad argument");
    rowmap_decode_kernel<<<(B + 127) / 128, 128, 0, st>>>(rm.segs, rm.row_slot, rm.row_pos, len, sstate, rows_state, slot0, B);
    B2_LAUNCH_CHECK();
    return 0;
}

}  // namespace b2
