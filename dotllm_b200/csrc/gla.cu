// Gated linear attention: a matrix-valued state per (sequence, head) that decays per key channel.
//
//   alpha_t = sigmoid(z_t)^(1/tau)                      (one decay per key channel, in (0, 1))
//   S_t     = diag(alpha_t) S_(t-1) + k_t v_t^T          (S: [key channels, value channels])
//   o_t     = S_t^T (q_t * q_scale)
//
// followed, in a second kernel, by an RMS norm of every head's o_t over its value channels, a gain
// shared by the heads, and a gate silu(g_t).  State, decays (through log sigmoid, so that a tiny
// sigmoid does not lose its digits before the root is taken), the recurrence and the norm are float32
// whatever the storage type of q, k, v, z and g.
//
// The scan walks a sequence's new tokens in order, starting from the state that the sequence's slot
// holds and leaving the new state there: a prompt, a part of a prompt and a single decoded token are
// the same loop, so a position's result does not depend on how its sequence was cut into steps.  A
// block owns GLA_COLS value channels of one (sequence, head): columns of S never mix, so blocks need
// nothing from each other.  GLA_SPLIT neighbouring lanes share a column, each holding every
// GLA_SPLIT-th key channel of it in registers; their partial sums of o meet by shuffles.  The token's
// q, k and decays are staged in shared memory (two buffers, one barrier per token) while the loads
// of the next token are in flight.
#include "common.cuh"

#define GLA_COLS 32
#define GLA_SPLIT 8
#define GLA_THREADS (GLA_COLS * GLA_SPLIT)
#define GLA_MAX_DIM GLA_THREADS          // key channels per head that the scan takes

template <typename T, int ROWS>
__global__ void __launch_bounds__(GLA_THREADS)
gla_scan_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, int ld,
                const float* __restrict__ z, int z_stride, const float* __restrict__ z_bias,
                const int32_t* __restrict__ cu_new, const int32_t* __restrict__ slots, float* __restrict__ state,
                int n_slots, float* __restrict__ out, int out_stride, int H, int dim, int vdim, float q_scale,
                float inv_tau) {
    __shared__ float sq[2][GLA_MAX_DIM], sk[2][GLA_MAX_DIM], sa[2][GLA_MAX_DIM];
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int tid = threadIdx.x, r = tid % GLA_SPLIT;
    const int col = blockIdx.x * GLA_COLS + tid / GLA_SPLIT;
    const bool col_ok = col < vdim;
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const int slot = slots[b];
    if (slot < 0 || slot >= n_slots || t0 >= t1) return;       // uniform over the block
    float* S = state + ((size_t)slot * H + h) * dim * vdim;
    float s[ROWS];
#pragma unroll
    for (int m = 0; m < ROWS; ++m) {
        const int i = r + GLA_SPLIT * m;
        s[m] = (i < dim && col_ok) ? S[(size_t)i * vdim + col] : 0.f;
    }
    float rq = 0.f, rk = 0.f, rz = 0.f, rv = 0.f;
    const bool loader = tid < dim;
    {
        const size_t row = (size_t)t0;
        if (loader) {
            rq = dl_to_f32<T>(q[row * ld + h * dim + tid]);
            rk = dl_to_f32<T>(k[row * ld + h * dim + tid]);
            rz = z[row * z_stride + h * dim + tid] + z_bias[h * dim + tid];
        }
        if (col_ok) rv = dl_to_f32<T>(v[row * ld + h * vdim + col]);
    }
    int buf = 0;
    for (int t = t0; t < t1; ++t) {
        if (loader) {
            sq[buf][tid] = rq * q_scale;
            sk[buf][tid] = rk;
            const float log_sigmoid = fminf(rz, 0.f) - log1pf(expf(-fabsf(rz)));
            sa[buf][tid] = expf(log_sigmoid * inv_tau);
        }
        const float vt = rv;
        __syncthreads();
        if (t + 1 < t1) {
            const size_t row = (size_t)(t + 1);
            if (loader) {
                rq = dl_to_f32<T>(q[row * ld + h * dim + tid]);
                rk = dl_to_f32<T>(k[row * ld + h * dim + tid]);
                rz = z[row * z_stride + h * dim + tid] + z_bias[h * dim + tid];
            }
            if (col_ok) rv = dl_to_f32<T>(v[row * ld + h * vdim + col]);
        }
        float o = 0.f;
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
            const int i = r + GLA_SPLIT * m;
            if (i < dim) {
                s[m] = sa[buf][i] * s[m] + sk[buf][i] * vt;
                o += s[m] * sq[buf][i];
            }
        }
        o += __shfl_xor_sync(0xffffffffu, o, 1);
        o += __shfl_xor_sync(0xffffffffu, o, 2);
        o += __shfl_xor_sync(0xffffffffu, o, 4);
        if (r == 0 && col_ok) out[(size_t)t * out_stride + h * vdim + col] = o;
        buf ^= 1;
    }
    if (col_ok) {
#pragma unroll
        for (int m = 0; m < ROWS; ++m) {
            const int i = r + GLA_SPLIT * m;
            if (i < dim) S[(size_t)i * vdim + col] = s[m];
        }
    }
}

template <typename T>
static int launch_scan(const void* q, const void* k, const void* v, int ld, const float* z, int z_stride, const float* z_bias,
                       const int32_t* cu_new, const int32_t* slots, float* state, int n_slots, float* out, int out_stride,
                       int n_seqs, int H, int dim, int vdim, float q_scale, float inv_tau, cudaStream_t s) {
    const dim3 grid((vdim + GLA_COLS - 1) / GLA_COLS, H, n_seqs), block(GLA_THREADS);
    const int rows = (dim + GLA_SPLIT - 1) / GLA_SPLIT;
    cudaError_t e;
#define GLA_LAUNCH(R)                                                                                                   \
    e = dl_launch_dependent(gla_scan_kernel<T, R>, grid, block, 0, s, (const T*)q, (const T*)k, (const T*)v, ld,        \
                            z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride, H, dim, vdim, \
                            q_scale, inv_tau)
    if (rows <= 4) GLA_LAUNCH(4);
    else if (rows <= 8) GLA_LAUNCH(8);
    else if (rows <= 16) GLA_LAUNCH(16);
    else GLA_LAUNCH(32);
#undef GLA_LAUNCH
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "gla_scan: %s", cudaGetErrorString(e));
    return DL_OK;
}

// q, k [tokens, H*dim] and v [tokens, H*vdim]: views with the common row stride ld (columns of one projection);
// z float32 [tokens, H*dim] (decay logits before the bias), rows z_stride apart; z_bias float32 [H*dim];
// cu_new int32 [n_seqs + 1] (offsets of each sequence's tokens among the step's rows); slots int32 [n_seqs];
// state float32 [n_slots, H, dim, vdim], read and updated; out float32 [tokens, H*vdim], rows out_stride apart.
extern "C" int dl_gla_scan(const void* q, const void* k, const void* v, int ld, const float* z, int z_stride,
                           const float* z_bias, int dtype, const int32_t* cu_new, const int32_t* slots, float* state,
                           int n_slots, float* out, int out_stride, int n_seqs, int H, int dim, int vdim, float q_scale,
                           float tau, void* stream) {
    DL_REQUIRE(n_seqs >= 0 && H > 0 && dim > 0 && vdim > 0 && n_slots > 0, "gla_scan: bad sizes");
    DL_REQUIRE(dim <= GLA_MAX_DIM, "gla_scan: %d key channels per head, the kernel takes up to %d", dim, GLA_MAX_DIM);
    DL_REQUIRE(tau > 0.f, "gla_scan: tau must be positive");
    DL_REQUIRE(out_stride >= H * vdim && z_stride >= H * dim, "gla_scan: rows overlap");
    if (n_seqs == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_F32)
        return launch_scan<float>(q, k, v, ld, z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride, n_seqs, H,
                                  dim, vdim, q_scale, 1.0f / tau, s);
    if (dtype == DL_BF16)
        return launch_scan<__nv_bfloat16>(q, k, v, ld, z, z_stride, z_bias, cu_new, slots, state, n_slots, out, out_stride,
                                          n_seqs, H, dim, vdim, q_scale, 1.0f / tau, s);
    return dl_fail(DL_ERR_UNSUPPORTED, "gla_scan: dtype %d", dtype);
}

// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * gain[:] * silu(g[t, h, :]): one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const T* __restrict__ g, int g_stride,
                      const float* __restrict__ gain, T* __restrict__ out, int out_stride, int rows, int H, int vdim,
                      float eps) {
    dl_launch_dependents();
    dl_grid_dependency_wait();
    const int lane = threadIdx.x & 31;
    const long idx = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (idx >= (long)rows * H) return;
    const int t = (int)(idx / H), h = (int)(idx % H);
    const float* orow = o + (size_t)t * o_stride + (size_t)h * vdim;
    float ss = 0.f;
    for (int j = lane; j < vdim; j += 32) ss += orow[j] * orow[j];
    ss = dl_warp_sum(ss);
    const float scale = 1.0f / sqrtf(ss / (float)vdim + eps);
    const T* grow = g + (size_t)t * g_stride + (size_t)h * vdim;
    T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
    for (int j = lane; j < vdim; j += 32) {
        const float gate = dl_to_f32<T>(grow[j]);
        dst[j] = dl_from_f32<T>(orow[j] * scale * gain[j] * (gate * (1.0f / (1.0f + expf(-gate)))));
    }
}

extern "C" int dl_head_norm_gate(const float* o, int o_stride, const void* g, int g_stride, const float* gain, void* out,
                                 int out_stride, int dtype, int rows, int H, int vdim, float eps, void* stream) {
    DL_REQUIRE(rows >= 0 && H > 0 && vdim > 0 && eps > 0.f, "head_norm_gate: bad arguments");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const long warps = (long)rows * H;
    const dim3 grid((unsigned)((warps + 3) / 4)), block(128);
    cudaError_t e;
    if (dtype == DL_F32)
        e = dl_launch_dependent(head_norm_gate_kernel<float>, grid, block, 0, s, o, o_stride, (const float*)g, g_stride, gain,
                                (float*)out, out_stride, rows, H, vdim, eps);
    else if (dtype == DL_BF16)
        e = dl_launch_dependent(head_norm_gate_kernel<__nv_bfloat16>, grid, block, 0, s, o, o_stride, (const __nv_bfloat16*)g,
                                g_stride, gain, (__nv_bfloat16*)out, out_stride, rows, H, vdim, eps);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "head_norm_gate: dtype %d", dtype);
    if (e != cudaSuccess) return dl_fail(DL_ERR_LAUNCH, "head_norm_gate: %s", cudaGetErrorString(e));
    return DL_OK;
}
