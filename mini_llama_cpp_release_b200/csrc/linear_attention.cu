// Gated linear attention: a matrix memory per head with a decay per key channel.
//
//   a_t = sigmoid(z_t)^(1/tau) = exp(logsigmoid(z_t) / tau)              (per head and key channel, float32)
//   S_t = diag(a_t) S_{t-1} + k_t v_tᵀ,     o_t = S_tᵀ (q_t · dim^-1/2)   (S: [dim][vdim] per head, float32)
//
// The state starts at zero, lives in float32 and is carried per sequence in a slot's row; decays, their logarithms
// and everything else that enters the recurrence are float32 whatever the engine's type.
//
// The walk: a block owns (sequence, head, 32 columns of S).  Eight neighbouring lanes share a column and hold every
// eighth row of it in registers; tokens arrive sixteen at a time through shared memory (q scaled, k, the decays
// already exponentiated), so the dependent chain per token is one multiply-add per held row, one more for the
// output, and three shuffles.  State layout in a slot's row: [head][column][row] (a column's rows side by side).
#include "common.cuh"

namespace mlc {

constexpr int GLA_COLS = 32;       // columns of S per block
constexpr int GLA_SPLIT = 8;       // lanes per column
constexpr int GLA_CHUNK = 16;      // tokens staged at a time

struct GlaArgs {
    const float* proj;          // rows of the input product
    long long proj_stride;
    int q_col, k_col, v_col;
    const float* z;             // [n][H*dim] decay logits without their bias
    const float* z_bias;        // [H*dim] or null
    float inv_tau;
    float q_scale;
    float* state;               // [slots][H*vdim*dim]
    long long state_stride;
    const int* slots;
    const int* cu_seqlens;
    float* out;                 // [n][H*vdim]
    int H, dim, vdim;
};

__device__ __forceinline__ float decay_of(float z, float inv_tau) {
    // logsigmoid(z) = min(z, 0) - log1p(exp(-|z|))
    const float ls = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
    return expf(ls * inv_tau);
}

template <int ROWS>       // rows of a column one lane holds: dim <= 8 * ROWS
__global__ void __launch_bounds__(GLA_COLS * GLA_SPLIT)
gla_walk_kernel(GlaArgs a) {
    extern __shared__ float sh[];
    const int dim = a.dim, vdim = a.vdim;
    float* qs = sh;                                  // [CHUNK][dim]
    float* ks = qs + GLA_CHUNK * dim;
    float* as = ks + GLA_CHUNK * dim;
    float* vs = as + GLA_CHUNK * dim;                // [CHUNK][GLA_COLS]
    const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * GLA_COLS;
    const int r = threadIdx.x % GLA_SPLIT, c = threadIdx.x / GLA_SPLIT;
    const int col = col0 + c;
    const bool col_ok = col < vdim;
    const int t0 = a.cu_seqlens[seq], t1 = a.cu_seqlens[seq + 1];
    float* S_row = a.state + (long long)a.slots[seq] * a.state_stride + ((long long)head * vdim + (col_ok ? col : 0)) * dim;
    float S[ROWS];
#pragma unroll
    for (int i = 0; i < ROWS; ++i) {
        const int row = i * GLA_SPLIT + r;
        S[i] = (col_ok && row < dim) ? S_row[row] : 0.0f;
    }
    for (int c0 = t0; c0 < t1; c0 += GLA_CHUNK) {
        const int n_here = min(GLA_CHUNK, t1 - c0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < n_here * dim; idx += blockDim.x) {
            const int tt = idx / dim, d = idx % dim;
            const float* row = a.proj + (long long)(c0 + tt) * a.proj_stride;
            qs[idx] = row[a.q_col + head * dim + d] * a.q_scale;
            ks[idx] = row[a.k_col + head * dim + d];
            const int zc = head * dim + d;
            as[idx] = decay_of(a.z[(long long)(c0 + tt) * a.H * dim + zc] + (a.z_bias != nullptr ? a.z_bias[zc] : 0.0f), a.inv_tau);
        }
        for (int idx = threadIdx.x; idx < n_here * GLA_COLS; idx += blockDim.x) {
            const int tt = idx / GLA_COLS, cc = idx % GLA_COLS;
            vs[idx] = (col0 + cc < vdim) ? a.proj[(long long)(c0 + tt) * a.proj_stride + a.v_col + head * vdim + col0 + cc] : 0.0f;
        }
        __syncthreads();
        for (int tt = 0; tt < n_here; ++tt) {
            const float v = vs[tt * GLA_COLS + c];
            const float* q = qs + tt * dim;
            const float* k = ks + tt * dim;
            const float* al = as + tt * dim;
            float acc = 0.0f;
#pragma unroll
            for (int i = 0; i < ROWS; ++i) {
                const int row = i * GLA_SPLIT + r;
                if (row < dim) {
                    S[i] = fmaf(al[row], S[i], k[row] * v);
                    acc = fmaf(S[i], q[row], acc);
                }
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (r == 0 && col_ok) a.out[(long long)(c0 + tt) * a.H * vdim + head * vdim + col] = acc;
        }
    }
    if (col_ok) {
#pragma unroll
        for (int i = 0; i < ROWS; ++i) {
            const int row = i * GLA_SPLIT + r;
            if (row < dim) S_row[row] = S[i];
        }
    }
}

}  // namespace mlc

using namespace mlc;

// proj: float32 rows (stride proj_stride) holding q (H x dim) at q_col, k (H x dim) at k_col, v (H x vdim) at v_col.
// z: float32 [n][H*dim] decay logits, z_bias [H*dim] or null.  state: float32, a slot's row holds H*vdim*dim floats.
// out: float32 [n][H*vdim].
extern "C" int mlc_gla(const float* proj, long long proj_stride, int q_col, int k_col, int v_col, const float* z,
                       const float* z_bias, float tau, float* state, long long state_stride, const int* slots,
                       const int* cu_seqlens, int n_seqs, int n_tokens, int H, int dim, int vdim, float* out, void* stream) {
    if (n_seqs <= 0 || n_tokens <= 0) return 0;
    if (H <= 0 || dim <= 0 || dim > 256 || vdim <= 0 || !(tau > 0.0f) || n_seqs > 65535) return MLC_ERR_BAD_SIZE;
    GlaArgs a{proj, proj_stride, q_col, k_col, v_col, z, z_bias, 1.0f / tau, 1.0f / sqrtf((float)dim), state, state_stride,
              slots, cu_seqlens, out, H, dim, vdim};
    const dim3 grid(H, n_seqs, (vdim + GLA_COLS - 1) / GLA_COLS);
    const size_t smem = (size_t)(3 * GLA_CHUNK * dim + GLA_CHUNK * GLA_COLS) * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (dim <= 32)
        gla_walk_kernel<4><<<grid, GLA_COLS * GLA_SPLIT, smem, s>>>(a);
    else if (dim <= 64)
        gla_walk_kernel<8><<<grid, GLA_COLS * GLA_SPLIT, smem, s>>>(a);
    else if (dim <= 128)
        gla_walk_kernel<16><<<grid, GLA_COLS * GLA_SPLIT, smem, s>>>(a);
    else {
        static bool raised = false;                // 16 tokens of 3 x 256 floats pass the default 48 KB
        if (!raised) {
            cudaError_t e = cudaFuncSetAttribute(gla_walk_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
            if (e != cudaSuccess) return (int)e;
            raised = true;
        }
        gla_walk_kernel<32><<<grid, GLA_COLS * GLA_SPLIT, smem, s>>>(a);
    }
    MLC_LAUNCH_CHECK();
    return 0;
}
