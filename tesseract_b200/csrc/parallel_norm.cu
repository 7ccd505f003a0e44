// The residual sum and the norms of a block whose mixer and feed-forward both read the same stream.
//
//   tb_sum_norms    c = res [+ (upd_a [+ upd_b])]  (32-bit; stored to res_out when an update is given)
//                   y1 = round(c * rsqrt(mean(c^2) + eps) * w1)
//                   y2 = round(c * rsqrt(mean(c^2) + eps) * w2)      (when w2 / y2 are given)
//                   Two RMS norms of one row share the row's statistic and differ in their weights only, so the
//                   row is read once and both outputs leave in one pass.
//   tb_sum_concat   out[t, 0 : width] = round(res + (upd_a + upd_b)),  out[t, width : 2 width] = round(origin):
//                   the pending sum of the stream beside a second stream, as the operand of one product.
//
// The stream and its updates are 32-bit; the outputs are 32-bit or bfloat16.  One block per row, the row kept in
// shared memory between the two passes; block size and reduction tree follow from the width alone, so a row's
// result does not depend on the batch around it.
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void store4(T* p, const float* v);
template <>
__device__ __forceinline__ void store4<float>(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}
__device__ __forceinline__ void load4(const float* p, float* v) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}

// VEC: four numbers a thread and iteration (width a multiple of four, buffers 16-byte aligned).
template <typename T, bool VEC>
__global__ void __launch_bounds__(1024)
sum_norms_kernel(const float* __restrict__ res, const float* __restrict__ upd_a, const float* __restrict__ upd_b,
                 const float* __restrict__ w1, T* __restrict__ y1, const float* __restrict__ w2, T* __restrict__ y2,
                 float* __restrict__ res_out, int width, float eps) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();                                   // the stream and its updates come from kernels in front
    const int64_t base = (int64_t)blockIdx.x * width;
    float ss = 0.0f;
    if (VEC) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {
            float v[4];
            load4(res + base + j, v);
            if (upd_a != nullptr) {
                float u[4];
                load4(upd_a + base + j, u);
                if (upd_b != nullptr) {
                    float t[4];
                    load4(upd_b + base + j, t);
#pragma unroll
                    for (int e = 0; e < 4; ++e) u[e] += t[e];
                }
#pragma unroll
                for (int e = 0; e < 4; ++e) v[e] += u[e];
                store4<float>(res_out + base + j, v);
            }
            store4<float>(row_cache + j, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss = fmaf(v[e], v[e], ss);
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            float v = res[base + j];
            if (upd_a != nullptr) {
                float u = upd_a[base + j];
                if (upd_b != nullptr) u += upd_b[base + j];
                v += u;
                res_out[base + j] = v;
            }
            row_cache[j] = v;
            ss = fmaf(v, v, ss);
        }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    if (VEC) {
        for (int j = threadIdx.x * 4; j < width; j += blockDim.x * 4) {      // each thread rereads what it wrote
            float v[4], wv[4], o[4];
            load4(row_cache + j, v);
            load4(w1 + j, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) o[e] = v[e] * inv * wv[e];
            store4<T>(y1 + base + j, o);
            if (y2 != nullptr) {
                load4(w2 + j, wv);
#pragma unroll
                for (int e = 0; e < 4; ++e) o[e] = v[e] * inv * wv[e];
                store4<T>(y2 + base + j, o);
            }
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            const float v = row_cache[j] * inv;
            Elem<T>::store(y1 + base + j, v * w1[j]);
            if (y2 != nullptr) Elem<T>::store(y2 + base + j, v * w2[j]);
        }
    }
}

template <typename T>
int launch_norms(const float* res, const float* upd_a, const float* upd_b, const float* w1, void* y1, const float* w2,
                 void* y2, float* res_out, int rows, int width, float eps, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_BAD_SIZE;
    const uintptr_t bits = (uintptr_t)res | (uintptr_t)upd_a | (uintptr_t)upd_b | (uintptr_t)w1 | (uintptr_t)w2 |
                           (uintptr_t)y1 | (uintptr_t)y2 | (uintptr_t)res_out;
    const bool vec = width % 4 == 0 && bits % 16 == 0;      // (the width and the alignment alone decide)
    int threads;
    if (vec) threads = width / 4 >= 1024 ? 1024 : ((width / 4 + 31) / 32) * 32;
    else {
        threads = 32;
        while (threads < 512 && threads * 4 < width) threads <<= 1;
    }
    auto kernel = vec ? sum_norms_kernel<T, true> : sum_norms_kernel<T, false>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    cudaError_t launched = tb_launch_pdl(kernel, dim3(rows), dim3(threads), smem, stream, res, upd_a, upd_b, w1, (T*)y1,
                                         w2, (T*)y2, res_out, width, eps);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename T>
__global__ void sum_concat_kernel(const float* __restrict__ res, const float* __restrict__ upd_a,
                                  const float* __restrict__ upd_b, const float* __restrict__ origin,
                                  T* __restrict__ out, int width) {
    pdl_trigger();
    pdl_wait();
    const int64_t base = (int64_t)blockIdx.x * width;
    T* orow = out + (int64_t)blockIdx.x * 2 * width;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < width; j += gridDim.y * blockDim.x) {
        float v = res[base + j];
        if (upd_a != nullptr) {
            float u = upd_a[base + j];
            if (upd_b != nullptr) u += upd_b[base + j];
            v += u;
        }
        Elem<T>::store(orow + j, v);
        Elem<T>::store(orow + width + j, origin[base + j]);
    }
}

}  // namespace

// res, upd_a, upd_b, res_out: 32-bit [rows, width] (upd_b needs upd_a; res_out, which may alias res, is written
// when upd_a is given); w1, w2: 32-bit [width]; y1, y2: [rows, width] of y_dtype (w2 and y2 may both be null).
TB_EXPORT int tb_sum_norms(const float* res, const float* upd_a, const float* upd_b, const float* w1, void* y1,
                           const float* w2, void* y2, float* res_out, int rows, int width, float eps, int y_dtype,
                           cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1) return TB_ERR_BAD_SIZE;
    if (upd_a == nullptr && upd_b != nullptr) return TB_ERR_BAD_SIZE;
    if (upd_a != nullptr && res_out == nullptr) return TB_ERR_BAD_SIZE;
    if ((w2 == nullptr) != (y2 == nullptr)) return TB_ERR_BAD_SIZE;
    if (y_dtype == TB_F32)
        return launch_norms<float>(res, upd_a, upd_b, w1, y1, w2, y2, res_out, rows, width, eps, stream);
    if (y_dtype == TB_BF16)
        return launch_norms<__nv_bfloat16>(res, upd_a, upd_b, w1, y1, w2, y2, res_out, rows, width, eps, stream);
    return TB_ERR_BAD_DTYPE;
}

// out: [rows, 2 * width] of out_dtype, contiguous.
TB_EXPORT int tb_sum_concat(const float* res, const float* upd_a, const float* upd_b, const float* origin, void* out,
                            int rows, int width, int out_dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1) return TB_ERR_BAD_SIZE;
    if (upd_a == nullptr && upd_b != nullptr) return TB_ERR_BAD_SIZE;
    const int threads = 256;
    int by = (width + threads - 1) / threads;
    if (by > 32) by = 32;
    const dim3 grid(rows, by);
    cudaError_t launched;
    if (out_dtype == TB_F32)
        launched = tb_launch_pdl(sum_concat_kernel<float>, grid, dim3(threads), 0, stream, res, upd_a, upd_b, origin,
                                 (float*)out, width);
    else if (out_dtype == TB_BF16)
        launched = tb_launch_pdl(sum_concat_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, res, upd_a, upd_b,
                                 origin, (__nv_bfloat16*)out, width);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
