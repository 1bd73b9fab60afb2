// SwiGLU gating: out = gate * sigmoid(gate) * up, float32 arithmetic.
// Reference: native/kernels/swiglu_f32.cu:5-15 and the scalar CPU twin
// src/DotLLM.Cpu/Kernels/FusedOps.cs:69-78 (sigmoid = 1 / (1 + exp(-g))).
#include "common.cuh"
#include "gating.cuh"

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_kernel(const T* __restrict__ gate, const T* __restrict__ up, int in_stride, T* __restrict__ out,
              int rows, int width) {
    const size_t n = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, c = i - r * width;
        const float g = dl_to_f32<T>(gate[r * in_stride + c]);
        const float u = dl_to_f32<T>(up[r * in_stride + c]);
        out[i] = dl_from_f32<T>(g * (1.0f / (1.0f + expf(-g))) * u);
    }
}

// gate, up: [rows, width] views with a common row stride; out: contiguous [rows, width].
extern "C" int dl_swiglu(const void* gate, const void* up, int in_stride, void* out, int dtype, int rows,
                         int width, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && in_stride >= width, "swiglu: bad sizes");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == DL_F32)
        swiglu_kernel<float><<<blocks, 256, 0, s>>>((const float*)gate, (const float*)up, in_stride, (float*)out,
                                                    rows, width);
    else if (dtype == DL_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                            in_stride, (__nv_bfloat16*)out, rows, width);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "swiglu: dtype %d", dtype);
    DL_CHECK_LAUNCH("swiglu");
    return DL_OK;
}

// Other gatings of a feed-forward's two products, float32 arithmetic, chosen by `kind`:
//   1  gelu_tanh(g) * u,  gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
//   2  g' sigmoid(alpha g') (u' + 1)  with g' = min(g, limit), u' = clamp(u, -limit, limit)
// (kind 0 is the SwiGLU above.)  `limit` and `alpha` are parameters of kind 2.
template <typename T>
__global__ void __launch_bounds__(256)
gated_activation_kernel(const T* __restrict__ gate, const T* __restrict__ up, int in_stride, T* __restrict__ out,
                        int rows, int width, int kind, float limit, float alpha) {
    const size_t n = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, c = i - r * width;
        out[i] = dl_from_f32<T>(dl_gate_value(kind, dl_to_f32<T>(gate[r * in_stride + c]), dl_to_f32<T>(up[r * in_stride + c]),
                                              limit, alpha));
    }
}

extern "C" int dl_gated_activation(const void* gate, const void* up, int in_stride, void* out, int dtype, int rows,
                                   int width, int kind, float limit, float alpha, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && in_stride >= width && kind >= 0 && kind < GATE_KINDS && dl_gate_is_gated(kind), "gated_activation: bad arguments");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == DL_F32)
        gated_activation_kernel<float><<<blocks, 256, 0, s>>>((const float*)gate, (const float*)up, in_stride, (float*)out,
                                                              rows, width, kind, limit, alpha);
    else if (dtype == DL_BF16)
        gated_activation_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)gate, (const __nv_bfloat16*)up,
                                                                      in_stride, (__nv_bfloat16*)out, rows, width, kind, limit, alpha);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "gated_activation: dtype %d", dtype);
    DL_CHECK_LAUNCH("gated_activation");
    return DL_OK;
}

// An activation of one product (gating.cuh: the kinds that read no gate, e.g. relu(x)^2): out = act(x), float32 arithmetic.
// x: [rows, width] with rows in_stride apart; out: contiguous [rows, width].
template <typename T>
__global__ void __launch_bounds__(256)
unary_activation_kernel(const T* __restrict__ x, int in_stride, T* __restrict__ out, int rows, int width, int kind) {
    const size_t n = (size_t)rows * width;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / width, c = i - r * width;
        out[i] = dl_from_f32<T>(dl_gate_value(kind, 0.f, dl_to_f32<T>(x[r * in_stride + c]), 0.f, 0.f));
    }
}

extern "C" int dl_unary_activation(const void* x, int in_stride, void* out, int dtype, int rows, int width, int kind, void* stream) {
    DL_REQUIRE(rows >= 0 && width > 0 && in_stride >= width, "unary_activation: bad sizes");
    DL_REQUIRE(kind >= 0 && kind < GATE_KINDS && !dl_gate_is_gated(kind), "unary_activation: kind %d is no activation of one product", kind);
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t n = (size_t)rows * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == DL_F32)
        unary_activation_kernel<float><<<blocks, 256, 0, s>>>((const float*)x, in_stride, (float*)out, rows, width, kind);
    else if (dtype == DL_BF16)
        unary_activation_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)x, in_stride, (__nv_bfloat16*)out, rows, width, kind);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "unary_activation: dtype %d", dtype);
    DL_CHECK_LAUNCH("unary_activation");
    return DL_OK;
}

// Soft cap of float32 values in place: x = cap * tanh(x / cap) (logits that may not exceed +-cap).
__global__ void __launch_bounds__(256) softcap_kernel(float* __restrict__ x, size_t n, float cap) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        x[i] = cap * tanhf(x[i] / cap);
}

extern "C" int dl_softcap(float* x, long long n, float cap, void* stream) {
    DL_REQUIRE(n >= 0 && cap > 0.f, "softcap: the cap must be positive");
    if (n == 0) return DL_OK;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    softcap_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(x, (size_t)n, cap);
    DL_CHECK_LAUNCH("softcap");
    return DL_OK;
}

// A gate per (row, head) on rows of `heads` heads of `width` values, in place: o[t, h, :] *= sigmoid(gate[t, h]).
// gate: one logit per head in rows gate_stride apart, of o's dtype.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ o, int o_stride, const T* __restrict__ gate, int gate_stride, int rows, int heads, int width) {
    const size_t per_row = (size_t)heads * width, n = (size_t)rows * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t r = i / per_row, c = i - r * per_row;
        const float g = 1.0f / (1.0f + expf(-dl_to_f32<T>(gate[r * gate_stride + c / width])));
        T* p = o + r * o_stride + c;
        *p = dl_from_f32<T>(dl_to_f32<T>(*p) * g);
    }
}

// The same for bfloat16 rows that can be moved 16 bytes at a time (width a multiple of 8, 16-byte aligned rows): a thread
// takes eight values of one head and computes that head's sigmoid once.
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(__nv_bfloat16* __restrict__ o, int o_stride, const __nv_bfloat16* __restrict__ gate, int gate_stride, int rows,
                     int heads, int width) {
    const int units = width / 8, per_row = heads * units;
    const size_t n = (size_t)rows * per_row;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / per_row), c = (int)(i - (size_t)r * per_row);
        const int h = c / units, u = c - h * units;
        const float g = 1.0f / (1.0f + expf(-__bfloat162float(gate[(size_t)r * gate_stride + h])));
        uint4* p = reinterpret_cast<uint4*>(o + (size_t)r * o_stride + (size_t)h * width + u * 8);
        uint4 raw = *p;
        __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = __floats2bfloat162_rn(__low2float(v[e]) * g, __high2float(v[e]) * g);
        *p = raw;
    }
}

extern "C" int dl_head_gate(void* o, int o_stride, const void* gate, int gate_stride, int dtype, int rows, int heads, int width,
                            void* stream) {
    DL_REQUIRE(rows >= 0 && heads > 0 && width > 0 && o_stride >= heads * width && gate_stride >= heads, "head_gate: bad sizes");
    if (rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_BF16 && width % 8 == 0 && o_stride % 8 == 0 && ((uintptr_t)o % 16) == 0) {
        const size_t units = (size_t)rows * heads * (width / 8);
        const int vblocks = (int)((units + 255) / 256 < 148 * 16 ? (units + 255) / 256 : 148 * 16);
        head_gate_vec_kernel<<<vblocks, 256, 0, s>>>((__nv_bfloat16*)o, o_stride, (const __nv_bfloat16*)gate, gate_stride, rows, heads, width);
        DL_CHECK_LAUNCH("head_gate");
        return DL_OK;
    }
    const size_t n = (size_t)rows * heads * width;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    if (dtype == DL_F32)
        head_gate_kernel<float><<<blocks, 256, 0, s>>>((float*)o, o_stride, (const float*)gate, gate_stride, rows, heads, width);
    else if (dtype == DL_BF16)
        head_gate_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((__nv_bfloat16*)o, o_stride, (const __nv_bfloat16*)gate, gate_stride, rows, heads, width);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "head_gate: dtype %d", dtype);
    DL_CHECK_LAUNCH("head_gate");
    return DL_OK;
}
