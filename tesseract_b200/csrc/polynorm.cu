// The normalised-polynomial activation of a feed-forward.
//
//   tb_polynorm   y = a * N(z) + b * N(z^2) + c * N(z^3) + e,  N(v) = v / sqrt(mean(v^2) + eps) over the row,
//                 powers element by element; (a, b, c, e) are four 32-bit numbers on the device.
//
// One block per row.  The row is read once into shared memory (32-bit; in 16-byte packets where its width and
// alignment allow), the three sums of squares (of z, z^2 and z^3) are taken in 32-bit through one reduction tree that
// the width alone fixes, and the row is written once, rounded once (so y may be z itself).  Input and output share a type (32-bit or bfloat16).
#include "common.cuh"

namespace {

// Three sums at once through one tree (fixed by blockDim alone); every thread receives the results.
__device__ __forceinline__ void block_sum3(float& a, float& b, float& c, float (*scratch)[32]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    a = warp_sum(a);
    b = warp_sum(b);
    c = warp_sum(c);
    if (lane == 0) {
        scratch[0][warp] = a;
        scratch[1][warp] = b;
        scratch[2][warp] = c;
    }
    __syncthreads();
    a = warp_sum(lane < warps ? scratch[0][lane] : 0.0f);
    b = warp_sum(lane < warps ? scratch[1][lane] : 0.0f);
    c = warp_sum(lane < warps ? scratch[2][lane] : 0.0f);
}

// VEC: the row is moved in 16-byte packets (its width a multiple of the packet, rows aligned).
template <typename T, bool VEC>
__global__ void polynorm_kernel(const T* z, int64_t z_stride, const float* __restrict__ coefficients,
                                T* y, int64_t y_stride, int width, float eps) {
    extern __shared__ __align__(16) float row_cache[];
    __shared__ float scratch[3][32];
    constexpr int N = Packet<T>::N;
    pdl_trigger();
    pdl_wait();                                   // the rows come from the product in front
    const T* zr = z + (int64_t)blockIdx.x * z_stride;
    float s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    if (VEC) {
        for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {
            float v[N];
            Packet<T>::load(zr + j, v);
#pragma unroll
            for (int e = 0; e < N; e += 4)              // (four numbers a store: a quarter of the bank conflicts)
                *reinterpret_cast<float4*>(row_cache + j + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float v2 = v[e] * v[e], v3 = v2 * v[e];
                s1 = fmaf(v[e], v[e], s1);
                s2 = fmaf(v2, v2, s2);
                s3 = fmaf(v3, v3, s3);
            }
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            const float v = Elem<T>::load(zr + j);
            row_cache[j] = v;
            const float v2 = v * v, v3 = v2 * v;
            s1 = fmaf(v, v, s1);
            s2 = fmaf(v2, v2, s2);
            s3 = fmaf(v3, v3, s3);
        }
    }
    block_sum3(s1, s2, s3, scratch);
    const float n = (float)width;
    const float k1 = coefficients[0] / sqrtf(s1 / n + eps);
    const float k2 = coefficients[1] / sqrtf(s2 / n + eps);
    const float k3 = coefficients[2] / sqrtf(s3 / n + eps);
    const float k0 = coefficients[3];
    T* yr = y + (int64_t)blockIdx.x * y_stride;
    if (VEC) {
        for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {      // each thread rereads what it wrote
            float o[N];
#pragma unroll
            for (int e = 0; e < N; e += 4) {
                const float4 t = *reinterpret_cast<const float4*>(row_cache + j + e);
                o[e] = t.x; o[e + 1] = t.y; o[e + 2] = t.z; o[e + 3] = t.w;
            }
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float v = o[e];
                const float v2 = v * v;
                o[e] = k1 * v + k2 * v2 + k3 * (v2 * v) + k0;
            }
            Packet<T>::store(yr + j, o);
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) {
            const float v = row_cache[j];
            const float v2 = v * v;
            Elem<T>::store(yr + j, k1 * v + k2 * v2 + k3 * (v2 * v) + k0);
        }
    }
}

template <typename T, bool VEC>
int launch_kind(const void* z, int64_t z_stride, const float* coefficients, void* y, int64_t y_stride, int rows,
                int width, float eps, cudaStream_t stream) {
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) return TB_ERR_BAD_SIZE;
    int threads = 64;
    while (threads < 1024 && threads * 8 < width) threads <<= 1;     // chosen by the width alone
    auto kernel = polynorm_kernel<T, VEC>;
    if (smem > 40 * 1024) {       // (the static scratch counts against the 48 KB a kernel has without asking)
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    cudaError_t launched = tb_launch_pdl(kernel, dim3(rows), dim3(threads), smem, stream, (const T*)z, z_stride,
                                         coefficients, (T*)y, y_stride, width, eps);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename T>
int launch(const void* z, int64_t z_stride, const float* coefficients, void* y, int64_t y_stride, int rows, int width,
           float eps, cudaStream_t stream) {
    constexpr int N = Packet<T>::N;
    const bool vec = width % N == 0 && z_stride % N == 0 && y_stride % N == 0 &&
                     ((uintptr_t)z | (uintptr_t)y) % 16 == 0;
    if (vec) return launch_kind<T, true>(z, z_stride, coefficients, y, y_stride, rows, width, eps, stream);
    return launch_kind<T, false>(z, z_stride, coefficients, y, y_stride, rows, width, eps, stream);
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
