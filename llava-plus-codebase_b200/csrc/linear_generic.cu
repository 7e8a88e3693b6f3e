// Linear layers on fp32 activations for shapes the tcgen05 GEMMs do not take (any M, N, K; fp32 or bf16 weights) and for
// true-fp32 compute: a weight-streaming row kernel for a handful of rows (decode) and a shared-memory tiled kernel for
// portions of a prompt. Accumulation is fp32 FMA in both; with round_a the activations are rounded to bf16 first, so the
// product is the bf16 x bf16 -> fp32 product the tensor-core path computes.
#include "common.cuh"
#include "kernels.h"

namespace b2 {
namespace {

__device__ __forceinline__ float ld_w(const float* p) { return *p; }
__device__ __forceinline__ float ld_w(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float lin_act(float v, int act) {
    switch (act) {
        case LIN_SILU: return v / (1.f + expf(-v));
        case LIN_SIGMOID: return 1.f / (1.f + expf(-v));
        case LIN_TANH: return tanhf(v);
        case LIN_RELU_SQ: { const float r = v > 0.f ? v : 0.f; return r * r; }
        default: return v;
    }
}
__device__ __forceinline__ void lin_store(float* o, float acc, const float* bias, int n, int act, float alpha, int accumulate) {
    float v = acc + (bias ? bias[n] : 0.f);
    v = alpha * lin_act(v, act);
    *o = accumulate ? (*o + v) : v;
}

__device__ __forceinline__ void ld_w4(const float* p, float (&w)[4]) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
}
__device__ __forceinline__ void ld_w4(const __nv_bfloat16* p, float (&w)[4]) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    w[0] = __uint_as_float(t.x << 16); w[1] = __uint_as_float(t.x & 0xffff0000u);
    w[2] = __uint_as_float(t.y << 16); w[3] = __uint_as_float(t.y & 0xffff0000u);
}

// ---- up to MR rows: one warp per output column, the weight row is read exactly once --------------------------------------
constexpr int MR = 8;
template <typename TW, bool VEC>
__global__ void __launch_bounds__(256) linear_rows_kernel(const float* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                                                          const float* __restrict__ bias, float* __restrict__ out, int64_t ld_out, int M, int N,
                                                          int K, int act, float alpha, int accumulate, int round_a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= N) return;
    const TW* w = W + (size_t)n * ldw;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) acc[m] = 0.f;
    if (VEC) {
        for (int k = lane * 4; k < K; k += 128) {
            float wv[4];
            ld_w4(w + k, wv);
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                if (m < M) {
                    float4 a = *reinterpret_cast<const float4*>(A + (size_t)m * lda + k);
                    if (round_a) { a.x = round_bf16(a.x); a.y = round_bf16(a.y); a.z = round_bf16(a.z); a.w = round_bf16(a.w); }
                    acc[m] = fmaf(a.x, wv[0], acc[m]); acc[m] = fmaf(a.y, wv[1], acc[m]);
                    acc[m] = fmaf(a.z, wv[2], acc[m]); acc[m] = fmaf(a.w, wv[3], acc[m]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            const float wv = ld_w(w + k);
#pragma unroll
            for (int m = 0; m < MR; ++m) {
                if (m < M) {
                    float a = A[(size_t)m * lda + k];
                    if (round_a) a = round_bf16(a);
                    acc[m] = fmaf(a, wv, acc[m]);
                }
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m) {
        float v = acc[m];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (lane == 0 && m < M) lin_store(out + (size_t)m * ld_out + n, v, bias, n, act, alpha, accumulate);
    }
}

// ---- portions of a prompt: 64 x 64 output tile, K in steps of 16, 4 x 4 outputs per thread -------------------------------
constexpr int TB = 64, TK = 16;
template <typename TW>
__global__ void __launch_bounds__(256) linear_tiled_kernel(const float* __restrict__ A, int64_t lda, const TW* __restrict__ W, int64_t ldw,
                                                           const float* __restrict__ bias, float* __restrict__ out, int64_t ld_out, int M, int N,
                                                           int K, int act, float alpha, int accumulate, int round_a) {
    __shared__ float As[TK][TB + 4];
    __shared__ float Ws[TK][TB + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * TB, n0 = blockIdx.x * TB;
    const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int idx = tid + e * 256;         // 64 rows x 16 k
            const int r = idx >> 4, kk = idx & 15;
            const int k = k0 + kk;
            float a = 0.f, w = 0.f;
            if (k < K) {
                if (m0 + r < M) { a = A[(size_t)(m0 + r) * lda + k]; if (round_a) a = round_bf16(a); }
                if (n0 + r < N) w = ld_w(W + (size_t)(n0 + r) * ldw + k);
            }
            As[kk][r] = a;
            Ws[kk][r] = w;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][tm]);
            const float4 w = *reinterpret_cast<const float4*>(&Ws[kk][tn]);
            const float av[4] = {a.x, a.y, a.z, a.w}, wv[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + tm + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) lin_store(out + (size_t)m * ld_out + n, acc[i][j], bias, n, act, alpha, accumulate);
        }
    }
}

template <typename TW>
int launch_linear(const LinearArgs& a, cudaStream_t st) {
    const TW* W = reinterpret_cast<const TW*>(a.W);
    if (a.M <= MR) {
        const bool vec = a.K % 4 == 0 && a.lda % 4 == 0 && a.ldw % 4 == 0 && (reinterpret_cast<uintptr_t>(a.A) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(a.W) & 15) == 0;
        dim3 grid((a.N + 7) / 8);
        if (vec)
            linear_rows_kernel<TW, true><<<grid, 256, 0, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, a.act, a.alpha,
                                                               a.accumulate, a.round_a);
        else
            linear_rows_kernel<TW, false><<<grid, 256, 0, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, a.act, a.alpha,
                                                                a.accumulate, a.round_a);
    } else {
        dim3 grid((a.N + TB - 1) / TB, (a.M + TB - 1) / TB);
        linear_tiled_kernel<TW><<<grid, 256, 0, st>>>(a.A, a.lda, W, a.ldw, a.bias, a.out, a.ld_out, a.M, a.N, a.K, a.act, a.alpha,
                                                      a.accumulate, a.round_a);
    }
    B2_LAUNCH_CHECK();
    return 0;
}
}  // namespace

int linear_f32(const LinearArgs& a, cudaStream_t st) {
    B2_CHECK_ARG(a.A && a.W && a.out && a.M > 0 && a.N > 0 && a.K > 0, "linear: bad argument (M=%d N=%d K=%d)", a.M, a.N, a.K);
    B2_CHECK_ARG(a.w_dtype == DT_F32 || a.w_dtype == DT_BF16, "linear: weights must be fp32 or bf16");
    return a.w_dtype == DT_F32 ? launch_linear<float>(a, st) : launch_linear<__nv_bfloat16>(a, st);
}

}  // namespace b2
