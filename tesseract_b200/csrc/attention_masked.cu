// Paged attention with 32-bit scores and weights, for mixers whose keys and values have widths of their own and
// whose mask, denominator and output are parameters:
//
//   mask     causal (every key up to the row's position), a sliding window of `mask_size` keys, or blocks: the
//            positions of a sequence are cut into consecutive blocks of `mask_size`, counted from position 0, and
//            a row sees the keys of its own block up to its own position;
//   sink     the softmax denominator has one more entry of score 0 that carries no value:
//            w_j = exp(s_j) / (1 + sum_j exp(s_j));
//   gate     the output is multiplied, element by element, by sigmoid(gate[row, head, :]).
//
// One warp per (query row, query head).  Keys are walked from the first visible one in blocks of 32, a lane a key:
// s_j = (q . k_j) * scale in 32-bit, a streaming softmax (running maximum m, sum l, accumulator acc; the sink is the
// start m = 0, l = 1), weights kept in 32-bit for the product with the values, lanes over the value's columns.  The
// order of every sum depends only on the row's position and the mask: not on the batch, on how the prompt was cut,
// or on the page ids.  A page is [G][page_size][d] keys followed by [G][page_size][dv] values.
//
// With block or window masks a row reads at most `mask_size` keys, so the work is linear in the rows of a step and
// the same kernel serves prompt portions and single decoded rows.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
enum MaskKind : int { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_BLOCKS = 2 };

template <typename T, int NCV, bool VEC>
__global__ void __launch_bounds__(kWarps * 32)
attention_masked_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate, int64_t gate_stride,
                        T* __restrict__ out, int64_t out_stride, const T* __restrict__ cache,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                        const int* __restrict__ block_table, int bt_stride, int heads, int kv_heads, int dim, int vdim,
                        int page_size, int mask_kind, int mask_size, int sink, float scale) {
    extern __shared__ float q_smem[];                 // kWarps * dim
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int head = blockIdx.y * kWarps + warp;
    if (head >= heads) return;                        // the whole warp leaves; no block-wide barrier below
    const int kv_head = head / (heads / kv_heads);
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    int first_key = 0;
    if (mask_kind == MASK_WINDOW) first_key = pos - mask_size + 1 > 0 ? pos - mask_size + 1 : 0;
    else if (mask_kind == MASK_BLOCKS) first_key = (pos / mask_size) * mask_size;

    float* qs = q_smem + warp * dim;
    const T* qrow = q + (int64_t)row * q_stride + (int64_t)head * dim;
    for (int i = lane; i < dim; i += 32) qs[i] = Elem<T>::load(qrow + i);
    __syncwarp();

    const int64_t page_elems = (int64_t)kv_heads * page_size * (dim + vdim);
    const T* kbase = cache + (int64_t)kv_head * page_size * dim;
    const T* vbase = cache + (int64_t)kv_heads * page_size * dim + (int64_t)kv_head * page_size * vdim;
    const int* table = block_table + (int64_t)seq * bt_stride;

    float m = sink ? 0.0f : -1.0e30f;
    float l = sink ? 1.0f : 0.0f;
    float acc[NCV];
#pragma unroll
    for (int c = 0; c < NCV; ++c) acc[c] = 0.0f;

    for (int key0 = first_key; key0 <= pos; key0 += 32) {
        const int key = key0 + lane;
        const bool valid = key <= pos;
        int64_t v_offset = 0;
        float s = -1.0e30f;
        if (valid) {
            const int64_t page = table[key / page_size];
            const int in_page = key % page_size;
            v_offset = page * page_elems + (int64_t)in_page * vdim;
            const T* kp = kbase + page * page_elems + (int64_t)in_page * dim;
            float dot = 0.0f;
            if (VEC) {
                constexpr int N = Packet<T>::N;
                float kv[N];
                for (int i = 0; i < dim; i += N) {
                    Packet<T>::load(kp + i, kv);
#pragma unroll
                    for (int e = 0; e < N; ++e) dot = fmaf(qs[i + e], kv[e], dot);
                }
            } else {
                for (int i = 0; i < dim; ++i) dot = fmaf(qs[i], Elem<T>::load(kp + i), dot);
            }
            s = dot * scale;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < NCV; ++c) acc[c] *= corr;
        const int keys_here = min(32, pos - key0 + 1);
        for (int j = 0; j < keys_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const int64_t off = __shfl_sync(0xffffffffu, v_offset, j);
            const T* vp = vbase + off;
#pragma unroll
            for (int c = 0; c < NCV; ++c) {
                const int col = c * 32 + lane;
                if (col < vdim) acc[c] = fmaf(pj, Elem<T>::load(vp + col), acc[c]);
            }
        }
        m = m_new;
    }
    const float denom = fmaxf(l, 1.0e-30f);
    T* orow = out + (int64_t)row * out_stride + (int64_t)head * vdim;
    const T* grow = gate == nullptr ? nullptr : gate + (int64_t)row * gate_stride + (int64_t)head * vdim;
#pragma unroll
    for (int c = 0; c < NCV; ++c) {
        const int col = c * 32 + lane;
        if (col < vdim) {
            float value = acc[c] / denom;
            if (grow != nullptr) value *= 1.0f / (1.0f + expf(-Elem<T>::load(grow + col)));
            Elem<T>::store(orow + col, value);
        }
    }
}

template <typename T, bool VEC>
int launch_vec(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
               const void* cache, const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
               int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind, int mask_size,
               int sink, float scale, cudaStream_t stream) {
    const dim3 grid(rows, (heads + kWarps - 1) / kWarps);
    const size_t smem = (size_t)kWarps * dim * sizeof(float);
#define TB_LAUNCH(NCV)                                                                                              \
    attention_masked_kernel<T, NCV, VEC><<<grid, kWarps * 32, smem, stream>>>(                                      \
        (const T*)q, q_stride, (const T*)gate, gate_stride, (T*)out, out_stride, (const T*)cache, positions,        \
        seq_of_row, block_table, bt_stride, heads, kv_heads, dim, vdim, page_size, mask_kind, mask_size, sink, scale)
    if (vdim <= 32) TB_LAUNCH(1);
    else if (vdim <= 64) TB_LAUNCH(2);
    else if (vdim <= 96) TB_LAUNCH(3);
    else if (vdim <= 128) TB_LAUNCH(4);
    else if (vdim <= 192) TB_LAUNCH(6);
    else TB_LAUNCH(8);
#undef TB_LAUNCH
    return tb_launch_status();
}

template <typename T>
int launch(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
           const void* cache, const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
           int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind, int mask_size, int sink,
           float scale, cudaStream_t stream) {
    // 16-byte key loads need every key row to start on a 16-byte boundary
    const bool vec = dim % Packet<T>::N == 0 && vdim % Packet<T>::N == 0 && (uintptr_t)cache % 16 == 0;
    if (vec)
        return launch_vec<T, true>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                   block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                   mask_size, sink, scale, stream);
    return launch_vec<T, false>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                mask_size, sink, scale, stream);
}

}  // namespace

// q: [rows, heads * dim] (row stride q_stride, elements); gate: null or [rows, heads * vdim] (row stride
// gate_stride); out: [rows, heads * vdim]; cache: this layer's pages.  mask_kind: 0 causal, 1 window, 2 blocks.
TB_EXPORT int tb_attention_masked(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out,
                                  int64_t out_stride, const void* cache, const int* positions, const int* seq_of_row,
                                  const int* block_table, int bt_stride, int rows, int heads, int kv_heads, int dim,
                                  int vdim, int page_size, int mask_kind, int mask_size, int sink, float scale,
                                  int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (dim < 1 || dim > 1024 || vdim < 1 || vdim > 256) return TB_ERR_BAD_SIZE;
    if (kv_heads < 1 || heads < 1 || heads % kv_heads != 0 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (mask_kind < MASK_CAUSAL || mask_kind > MASK_BLOCKS) return TB_ERR_BAD_SIZE;
    if (mask_kind != MASK_CAUSAL && mask_size < 1) return TB_ERR_BAD_SIZE;
    if ((heads + kWarps - 1) / kWarps > 65535) return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32)
        return launch<float>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row, block_table,
                             bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind, mask_size, sink, scale,
                             stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                     block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                     mask_size, sink, scale, stream);
    return TB_ERR_BAD_DTYPE;
}
