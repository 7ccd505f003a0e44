// The normalised-polynomial activation of a feed-forward.
//
//   tb_polynorm   y = a * N(z) + b * N(z^2) + c * N(z^3) + e,  N(v) = v / sqrt(mean(v^2) + eps) over the row,
//                 powers element by element; (a, b, c, e) are four 32-bit numbers on the device.
//
// One block per row.  The row is read once into shared memory (32-bit), the three sums of squares (of z, z^2 and
// z^3) are taken in 32-bit with a reduction tree that the width alone fixes, and the row is written once, rounded
// once (so y may be z itself).  Input and output share a type (32-bit or bfloat16).
#include "common.cuh"

namespace {

template <typename T>
__global__ void polynorm_kernel(const T* z, int64_t z_stride, const float* __restrict__ coefficients,
                                T* y, int64_t y_stride, int width, float eps) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float scratch[32];
    const T* zr = z + (int64_t)blockIdx.x * z_stride;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = Elem<T>::load(zr + j);
        row_cache[j] = v;
        const float v2 = v * v, v3 = v2 * v;
        s1 = fmaf(v, v, s1);
        s2 = fmaf(v2, v2, s2);
        s3 = fmaf(v3, v3, s3);
    }
    s1 = block_sum(s1, scratch);
    s2 = block_sum(s2, scratch);
    s3 = block_sum(s3, scratch);
    const float n = (float)width;
    const float k1 = coefficients[0] / sqrtf(s1 / n + eps);
    const float k2 = coefficients[1] / sqrtf(s2 / n + eps);
    const float k3 = coefficients[2] / sqrtf(s3 / n + eps);
    const float k0 = coefficients[3];
    T* yr = y + (int64_t)blockIdx.x * y_stride;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float v = row_cache[j];
        const float v2 = v * v;
        Elem<T>::store(yr + j, k1 * v + k2 * v2 + k3 * (v2 * v) + k0);
    }
}

template <typename T>
int launch(const void* z, int64_t z_stride, const float* coefficients, void* y, int64_t y_stride, int rows, int width,
           float eps, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 1024 && threads * 8 < width) threads <<= 1;
    auto kernel = polynorm_kernel<T>;
    if (smem > 48 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    kernel<<<rows, threads, smem, stream>>>((const T*)z, z_stride, coefficients, (T*)y, y_stride, width, eps);
    return tb_launch_status();
}

}  // namespace

TB_EXPORT int tb_polynorm(const void* z, int64_t z_stride, const float* coefficients, void* y, int64_t y_stride,
                          int rows, int width, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1) return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32) return launch<float>(z, z_stride, coefficients, y, y_stride, rows, width, eps, stream);
    if (dtype == TB_BF16) return launch<__nv_bfloat16>(z, z_stride, coefficients, y, y_stride, rows, width, eps, stream);
    return TB_ERR_BAD_DTYPE;
}
