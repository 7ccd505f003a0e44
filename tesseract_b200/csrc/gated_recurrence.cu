// An element-wise gated recurrence whose gates read only the current token (minGRU), with its output gate:
//
//   z_t = sigmoid(a_t + bz)                       a, u, g: the three projections of the row, side by side
//   c_t = u_t + bx + 1/2   where u_t + bx >= 0,   sigmoid(u_t + bx) below
//   S_t = (1 - z_t) * S_(t-1) + z_t * c_t         per channel; S lives in 32-bit in the request's state slot
//   y_t = S_t * silu(g_t)
//
// Everything but the projections is 32-bit.  A block owns 32 neighbouring channels of one sequence (a lane a
// channel, so rows are read in full 128-byte lines) and cuts the sequence's rows of this step into one run per
// warp.  Because S_t is affine in S_(t-1), a run is first reduced to the pair (A, B) with S_end = A * S_start + B
// (A the product of the (1 - z), B the run from a zero start); the warps' pairs are chained from the slot's state to
// give every run its start, and the run is then walked again with that start, writing y.  With one warp (steps of
// few rows) this is the plain walk.  The start state is read before, and the end state written after, everything
// else, by the warp that owns the last row.
#include "common.cuh"

namespace {

constexpr int kMaxWarps = 16;

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename TI, typename TO>
__global__ void __launch_bounds__(kMaxWarps * 32)
gated_recurrence_kernel(const TI* __restrict__ proj, int64_t proj_stride, const float* __restrict__ bias_z,
                        const float* __restrict__ bias_x, float* __restrict__ state, TO* __restrict__ out,
                        int64_t out_stride, const int* __restrict__ row_start, const int* __restrict__ state_slots,
                        int width) {
    __shared__ float run_a[kMaxWarps][32], run_b[kMaxWarps][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int seq = blockIdx.x;
    const int c = blockIdx.y * 32 + lane;
    const bool active = c < width;
    const int first_row = row_start[seq];
    const int n = row_start[seq + 1] - first_row;
    const int per_warp = (n + warps - 1) / warps;
    const int lo = min(n, warp * per_warp), hi = min(n, lo + per_warp);
    float* slot_state = state + (int64_t)state_slots[seq] * width;
    float s = active ? slot_state[c] : 0.0f;
    const float bz = active ? bias_z[c] : 0.0f, bx = active ? bias_x[c] : 0.0f;
    const TI* base = proj + (int64_t)first_row * proj_stride + c;

    if (warps > 1) {
        float a = 1.0f, b = 0.0f;
        if (active) {
            for (int t = lo; t < hi; ++t) {
                const TI* r = base + (int64_t)t * proj_stride;
                const float z = sigmoid_f32(Elem<TI>::load(r) + bz);
                const float u = Elem<TI>::load(r + width) + bx;
                const float cand = u >= 0.0f ? u + 0.5f : sigmoid_f32(u);
                const float keep = 1.0f - z;
                a *= keep;
                b = fmaf(z, cand, keep * b);
            }
        }
        run_a[warp][lane] = a;
        run_b[warp][lane] = b;
        __syncthreads();
        for (int k = 0; k < warp; ++k) s = fmaf(run_a[k][lane], s, run_b[k][lane]);
    }
    if (!active) return;
    for (int t = lo; t < hi; ++t) {
        const TI* r = base + (int64_t)t * proj_stride;
        const float z = sigmoid_f32(Elem<TI>::load(r) + bz);
        const float u = Elem<TI>::load(r + width) + bx;
        const float g = Elem<TI>::load(r + 2 * (int64_t)width);
        const float cand = u >= 0.0f ? u + 0.5f : sigmoid_f32(u);
        s = fmaf(z, cand, (1.0f - z) * s);
        Elem<TO>::store(out + (int64_t)(first_row + t) * out_stride + c, s * (g * sigmoid_f32(g)));
    }
    if (hi == n && lo < n) slot_state[c] = s;
}

template <typename TI, typename TO>
int launch(const void* proj, int64_t proj_stride, const float* bias_z, const float* bias_x, float* state, void* out,
           int64_t out_stride, const int* row_start, const int* state_slots, int num_seqs, int width, int max_new,
           cudaStream_t stream) {
    int warps = 1;
    while (warps < kMaxWarps && warps * 16 < max_new) warps <<= 1;     // runs of at least 16 rows
    const dim3 grid(num_seqs, (width + 31) / 32);
    gated_recurrence_kernel<TI, TO><<<grid, warps * 32, 0, stream>>>((const TI*)proj, proj_stride, bias_z, bias_x, state,
                                                                     (TO*)out, out_stride, row_start, state_slots,
                                                                     width);
    return tb_launch_status();
}

}  // namespace

// proj: [rows, 3 * width] (a | u | g) with row stride proj_stride, of in_dtype; bias_z, bias_x: 32-bit [width];
// state: 32-bit [slots, width]; out: [rows, width] of out_dtype; max_new: the most rows any sequence brings (it
// chooses the number of runs, never the values beyond rounding).
TB_EXPORT int tb_gated_recurrence(const void* proj, int64_t proj_stride, int in_dtype, const float* bias_z,
                                  const float* bias_x, float* state, void* out, int64_t out_stride, int out_dtype,
                                  const int* row_start, const int* state_slots, int num_seqs, int width, int max_new,
                                  cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    if (width < 1 || (width + 31) / 32 > 65535) return TB_ERR_BAD_SIZE;
    if (in_dtype == TB_F32 && out_dtype == TB_F32)
        return launch<float, float>(proj, proj_stride, bias_z, bias_x, state, out, out_stride, row_start, state_slots,
                                    num_seqs, width, max_new, stream);
    if (in_dtype == TB_F32 && out_dtype == TB_BF16)
        return launch<float, __nv_bfloat16>(proj, proj_stride, bias_z, bias_x, state, out, out_stride, row_start,
                                            state_slots, num_seqs, width, max_new, stream);
    if (in_dtype == TB_BF16 && out_dtype == TB_BF16)
        return launch<__nv_bfloat16, __nv_bfloat16>(proj, proj_stride, bias_z, bias_x, state, out, out_stride, row_start,
                                                    state_slots, num_seqs, width, max_new, stream);
    return TB_ERR_BAD_DTYPE;
}
