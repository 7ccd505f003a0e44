// An element-wise gated recurrence whose gates read only the current token (minGRU), with its output gate:
//
//   z_t = sigmoid(a_t + bz)                       a, u, g: the three projections of the row, side by side
//   c_t = u_t + bx + 1/2   where u_t + bx >= 0,   sigmoid(u_t + bx) below
//   S_t = (1 - z_t) * S_(t-1) + z_t * c_t         per channel; S lives in 32-bit in the request's state slot
//   y_t = S_t * silu(g_t)
//
// Everything but the projections is 32-bit.  A block owns 16 neighbouring channels of one sequence (a half-warp of
// lanes, so rows are read in whole 64-byte pieces) and cuts the sequence's rows of this step into one run per
// half-warp, up to 64 runs: a prompt of one sequence still fills the machine (in steps of at most 16 rows a
// sequence a block owns 128 channels and one run).  Because S_t is affine in S_(t-1), a
// run is first reduced to the pair (A, B) with S_end = A * S_start + B (A the product of the (1 - z), B the run from
// a zero start); the runs' pairs are chained from the slot's state to give every run its start, and the run is then
// walked again with that start, writing y.  A sequence whose rows fit one run (a decoded row, a short portion) is
// walked once.  The start state is read before, and the end state written after, everything else, by the thread
// that owns the last row.
#include "common.cuh"

namespace {

constexpr int kChannels = 16;       // channels of a block that cuts its rows into runs
constexpr int kMaxRuns = 64;        // runs of rows of a block (threads = runs * channels)
constexpr int kWideChannels = 128;  // channels of a block in steps of few rows (one run: the plain walk)

// (the exponential and the division as single hardware approximations: two units in the last place each, far inside
// what a 32-bit result is asked to hold)
__device__ __forceinline__ float sigmoid_f32(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

template <typename TI, typename TO>
__global__ void __launch_bounds__(kMaxRuns * kChannels)
gated_recurrence_kernel(const TI* __restrict__ proj, int64_t proj_stride, const float* __restrict__ bias_z,
                        const float* __restrict__ bias_x, float* __restrict__ state, TO* __restrict__ out,
                        int64_t out_stride, const int* __restrict__ row_start, const int* __restrict__ state_slots,
                        int width, int chans) {
    __shared__ float run_a[kMaxRuns * kChannels], run_b[kMaxRuns * kChannels];
    pdl_trigger();
    pdl_wait();                                   // the projections and the row starts come from kernels in front
    const int ch = threadIdx.x % chans, run = threadIdx.x / chans, runs = blockDim.x / chans;
    const int seq = blockIdx.x;
    const int c = blockIdx.y * chans + ch;
    const bool active = c < width;
    const int first_row = row_start[seq];
    const int n = row_start[seq + 1] - first_row;
    const int per_run = (n + runs - 1) / runs;
    const int lo = min(n, run * per_run), hi = min(n, lo + per_run);
    float* slot_state = state + (int64_t)state_slots[seq] * width;
    float s = active ? slot_state[c] : 0.0f;
    const float bz = active ? bias_z[c] : 0.0f, bx = active ? bias_x[c] : 0.0f;
    const TI* base = proj + (int64_t)first_row * proj_stride + c;

    if (runs > 1 && n > per_run) {          // (the same for every thread of the block)
        float a = 1.0f, b = 0.0f;
        if (active) {
#pragma unroll 4
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
        run_a[run * chans + ch] = a;
        run_b[run * chans + ch] = b;
        __syncthreads();
        for (int k = 0; k < run; ++k) s = fmaf(run_a[k * chans + ch], s, run_b[k * chans + ch]);
    }
    if (!active) return;
#pragma unroll 4
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
    int runs = 1;
    while (runs < kMaxRuns && runs * 16 < max_new) runs <<= 1;          // runs of at least 16 rows
    const int chans = runs == 1 ? kWideChannels : kChannels;
    const dim3 grid(num_seqs, (width + chans - 1) / chans);
    cudaError_t launched = tb_launch_pdl(gated_recurrence_kernel<TI, TO>, grid, dim3(runs * chans), 0, stream,
                                         (const TI*)proj, proj_stride, bias_z, bias_x, state, (TO*)out, out_stride,
                                         row_start, state_slots, width, chans);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
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
    if (width < 1 || (width + kChannels - 1) / kChannels > 65535) return TB_ERR_BAD_SIZE;      // (grid.y)
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
