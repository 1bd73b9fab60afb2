// Row gather: token embedding lookup into the float32 residual stream, and selection of
// the rows whose logits are wanted.
//
// Role of the reference's embedding_lookup_* kernels (native/kernels/embedding.cu:30-46,
// native/kernels/embedding_f32out.cu:10-70): one block per output row, the row copied
// with widening to float32 (or kept in bfloat16, for rows of activations that go on to a product).
#include "common.cuh"

template <typename T, typename TOut>
__global__ void __launch_bounds__(256)
gather_rows_kernel(const T* __restrict__ table, int table_stride, const int32_t* __restrict__ ids,
                   TOut* __restrict__ out, int width, int n_table_rows) {
    dl_launch_dependents();
    const int row = blockIdx.x;
    const int id = ids[row];
    TOut* dst = out + (size_t)row * width;
    if (id < 0 || id >= n_table_rows) {          // the host validates ids; never read outside the table
        for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = dl_from_f32<TOut>(0.f);
        return;
    }
    const T* src = table + (size_t)id * table_stride;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = dl_from_f32<TOut>(dl_to_f32<T>(src[c]));
}

// out[r, :] = table[ids[r], :] as `out_dtype`.  table: [n_table_rows, width] of `dtype`, rows
// table_stride elements apart; out: contiguous [n_rows, width], float32 or (from a bfloat16 table) bfloat16.
extern "C" int dl_gather_rows(const void* table, int dtype, int table_stride, const int32_t* ids, void* out, int out_dtype,
                              int n_rows, int width, int n_table_rows, void* stream) {
    DL_REQUIRE(n_rows >= 0 && width > 0 && n_table_rows > 0 && table_stride >= width,
               "gather_rows: bad sizes rows=%d width=%d table=%d stride=%d", n_rows, width, n_table_rows, table_stride);
    if (n_rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_F32 && out_dtype == DL_F32)
        gather_rows_kernel<float, float><<<n_rows, 256, 0, s>>>((const float*)table, table_stride, ids, (float*)out, width, n_table_rows);
    else if (dtype == DL_BF16 && out_dtype == DL_F32)
        gather_rows_kernel<__nv_bfloat16, float><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, table_stride, ids, (float*)out,
                                                                         width, n_table_rows);
    else if (dtype == DL_BF16 && out_dtype == DL_BF16)
        gather_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, table_stride, ids,
                                                                                 (__nv_bfloat16*)out, width, n_table_rows);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "gather_rows: from dtype %d to dtype %d", dtype, out_dtype);
    DL_CHECK_LAUNCH("gather_rows");
    return DL_OK;
}

// Token embedding plus a learned position vector: out[r, :] = table[ids[r], :] + positions[pos[r], :],
// the sum in float32.  One block per row.
template <typename T>
__global__ void __launch_bounds__(256)
embed_positions_kernel(const T* __restrict__ table, const T* __restrict__ pos_table, const int32_t* __restrict__ ids,
                       const int32_t* __restrict__ pos, float* __restrict__ out, int width, int n_table_rows,
                       int n_positions) {
    dl_launch_dependents();
    const int row = blockIdx.x;
    const int id = ids[row], p = pos[row];
    float* dst = out + (size_t)row * width;
    const bool ok = id >= 0 && id < n_table_rows && p >= 0 && p < n_positions;   // host-validated
    const T* a = table + (size_t)(ok ? id : 0) * width;
    const T* b = pos_table + (size_t)(ok ? p : 0) * width;
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = ok ? dl_to_f32<T>(a[c]) + dl_to_f32<T>(b[c]) : 0.f;
}

// table [n_table_rows, width], pos_table [n_positions, width] of `dtype`, both contiguous; out float32 [n_rows, width].
extern "C" int dl_embed_positions(const void* table, const void* pos_table, int dtype, const int32_t* ids,
                                  const int32_t* pos, float* out, int n_rows, int width, int n_table_rows,
                                  int n_positions, void* stream) {
    DL_REQUIRE(n_rows >= 0 && width > 0 && n_table_rows > 0 && n_positions > 0, "embed_positions: bad sizes");
    if (n_rows == 0) return DL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DL_F32)
        embed_positions_kernel<float><<<n_rows, 256, 0, s>>>((const float*)table, (const float*)pos_table, ids, pos, out, width,
                                                             n_table_rows, n_positions);
    else if (dtype == DL_BF16)
        embed_positions_kernel<__nv_bfloat16><<<n_rows, 256, 0, s>>>((const __nv_bfloat16*)table, (const __nv_bfloat16*)pos_table,
                                                                     ids, pos, out, width, n_table_rows, n_positions);
    else
        return dl_fail(DL_ERR_UNSUPPORTED, "embed_positions: dtype %d", dtype);
    DL_CHECK_LAUNCH("embed_positions");
    return DL_OK;
}
