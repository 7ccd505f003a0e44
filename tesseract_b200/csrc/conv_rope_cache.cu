// Short causal convolutions on projected queries, keys and values, the rotation of queries and keys, and the
// write of keys and values into the request's cache pages: what stands between an attention mixer's input
// projection and its attention kernel, in one pass over the projected rows.
//
// A projected row holds, side by side, H query heads of d numbers, G key heads of d numbers and G value heads of
// dv numbers (anything behind them in the row, an output gate for instance, is left alone).  Per channel c:
//
//   y[t] = sum_{j < J} taps[j, c] * u[t - (J - 1) + j]        (u = 0 before the sequence starts)
//
// where u at positions before this step's first token comes from the request's convolution state (the last J - 1
// projected rows, 32-bit, [slot][J - 1][channels]; position p of the request lies at index p - (begin - (J - 1))).
// Then, for queries and keys, the first `rot_dims` numbers of every head turn in pairs (2i, 2i + 1) by the angle
// position * inv_freq[i] (32-bit, sincosf); the rest of the head passes.  Queries go to q_out, keys and values
// into the pages: a page is [G][page_size][d] keys followed by [G][page_size][dv] values.
//
// All arithmetic is 32-bit; each stored value is rounded once.  A thread owns one pair of neighbouring channels
// of one row (or, in the packet kernel, one 16-byte packet of channels of a few rows in turn), and every channel's
// sum runs over its taps in the same order, so a row's values do not depend on the batch around it.
//
// The state is renewed (to the last J - 1 projected rows of the request) by tb_conv_state_update after the
// convolution of a step has read it, or, in a step where every sequence brings one row (`single` != 0), by the
// thread that owns the channel pair: there the only reader of a sequence's old state is that same thread.
#include "common.cuh"

namespace {

constexpr int kMaxTaps = 8;

struct ConvGeometry {
    int heads, kv_heads, dim, vdim;      // H, G, d, dv
    int rot_dims;                        // even, <= dim; 0: no rotation
    int taps;                            // J >= 1
    int page_size;
    int channels;                        // H*d + G*d + G*dv
    int q_pairs, k_pairs, v_pairs;       // pair slots per segment: heads * ceil(head size / 2)
};

template <typename T, bool SINGLE>
__global__ void __launch_bounds__(128)
conv_rope_cache_kernel(const T* __restrict__ proj, int64_t proj_stride, const float* __restrict__ taps,
                       float* __restrict__ state, T* __restrict__ q_out, int64_t q_stride, T* __restrict__ cache,
                       const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                       const int* __restrict__ row_start, const int* __restrict__ seq_begin,
                       const int* __restrict__ state_slots, const int* __restrict__ block_table, int bt_stride,
                       const float* __restrict__ inv_freq, ConvGeometry g, int write_kv) {
    pdl_trigger();
    pdl_wait();                                   // the projected rows and the step's metadata come from kernels in front
    const int row = blockIdx.x;
    const int slot_index = blockIdx.y * blockDim.x + threadIdx.x;
    const int total_pairs = g.q_pairs + g.k_pairs + g.v_pairs;
    if (slot_index >= total_pairs) return;
    // which segment, head and pair
    int segment, local, head_size, seg_offset;
    if (slot_index < g.q_pairs) {
        segment = 0; local = slot_index; head_size = g.dim; seg_offset = 0;
    } else if (slot_index < g.q_pairs + g.k_pairs) {
        segment = 1; local = slot_index - g.q_pairs; head_size = g.dim; seg_offset = g.heads * g.dim;
    } else {
        segment = 2; local = slot_index - g.q_pairs - g.k_pairs; head_size = g.vdim;
        seg_offset = (g.heads + g.kv_heads) * g.dim;
    }
    const int pairs_per_head = (head_size + 1) / 2;
    const int head = local / pairs_per_head;
    const int pair = local % pairs_per_head;
    const int e0 = 2 * pair;
    const bool has_second = e0 + 1 < head_size;
    const int c0 = seg_offset + head * head_size + e0;

    const int seq = seq_of_row[row];
    const int pos = positions[row];
    const int begin = seq_begin[seq];
    const int first_row = row_start[seq];
    const int slot = state_slots[seq];
    const int J = g.taps;
    float* st = state + (int64_t)slot * (J - 1) * g.channels;

    // the J projected values that end at this row, oldest first
    float u0[kMaxTaps], u1[kMaxTaps];
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < J) {
            const int p = pos - (J - 1) + j;
            float a = 0.0f, b = 0.0f;
            if (p >= begin) {
                const T* src = proj + (int64_t)(first_row + (p - begin)) * proj_stride + c0;
                a = Elem<T>::load(src);
                if (has_second) b = Elem<T>::load(src + 1);
            } else if (p >= 0) {
                const float* src = st + (int64_t)(p - (begin - (J - 1))) * g.channels + c0;
                a = src[0];
                if (has_second) b = src[1];
            }
            u0[j] = a;
            u1[j] = b;
        }
    }
    float y0 = 0.0f, y1 = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxTaps; ++j) {
        if (j < J) {
            y0 = fmaf(taps[(int64_t)j * g.channels + c0], u0[j], y0);
            if (has_second) y1 = fmaf(taps[(int64_t)j * g.channels + c0 + 1], u1[j], y1);
        }
    }
    if (SINGLE && J > 1) {
        // this thread is the only reader of these two channels of the sequence's state: shift it by one row
#pragma unroll
        for (int j = 1; j < kMaxTaps; ++j) {
            if (j < J) {
                float* dst = st + (int64_t)(j - 1) * g.channels + c0;
                dst[0] = u0[j];
                if (has_second) dst[1] = u1[j];
            }
        }
    }
    if (segment < 2 && e0 < g.rot_dims && has_second) {
        float sn, cs;
        sincosf((float)pos * inv_freq[pair], &sn, &cs);
        const float r0 = y0 * cs - y1 * sn;
        const float r1 = y1 * cs + y0 * sn;
        y0 = r0;
        y1 = r1;
    }
    if (segment == 0) {
        T* dst = q_out + (int64_t)row * q_stride + head * g.dim + e0;
        Elem<T>::store(dst, y0);
        if (has_second) Elem<T>::store(dst + 1, y1);
        return;
    }
    if (!write_kv) return;
    const int page = block_table[(int64_t)seq * bt_stride + pos / g.page_size];
    const int in_page = pos % g.page_size;
    const int64_t page_elems = (int64_t)g.kv_heads * g.page_size * (g.dim + g.vdim);
    T* dst = cache + (int64_t)page * page_elems;
    if (segment == 1) dst += ((int64_t)head * g.page_size + in_page) * g.dim + e0;
    else dst += (int64_t)g.kv_heads * g.page_size * g.dim + ((int64_t)head * g.page_size + in_page) * g.vdim + e0;
    Elem<T>::store(dst, y0);
    if (has_second) Elem<T>::store(dst + 1, y1);
}

// The same work in 16-byte packets, for head sizes that are multiples of a packet (8 bfloat16, 4 floats) and up to
// four taps: a thread owns one packet of channels for kRowTile neighbouring rows, holds that packet's taps in
// registers, and reads J packets per row (rows of this step) or J runs of 32-bit numbers (rows of the state).
constexpr int kRowTile = 4;

template <int N>
__device__ __forceinline__ void load_floats(const float* p, float* v) {
#pragma unroll
    for (int e = 0; e < N; e += 4) {
        const float4 t = *reinterpret_cast<const float4*>(p + e);
        v[e] = t.x; v[e + 1] = t.y; v[e + 2] = t.z; v[e + 3] = t.w;
    }
}
template <int N>
__device__ __forceinline__ void store_floats(float* p, const float* v) {
#pragma unroll
    for (int e = 0; e < N; e += 4) *reinterpret_cast<float4*>(p + e) = make_float4(v[e], v[e + 1], v[e + 2], v[e + 3]);
}

template <typename T, bool SINGLE, int J>
__global__ void __launch_bounds__(128)
conv_rope_cache_packets_kernel(const T* __restrict__ proj, int64_t proj_stride, const float* __restrict__ taps,
                               float* __restrict__ state, T* __restrict__ q_out, int64_t q_stride,
                               T* __restrict__ cache, const int* __restrict__ positions,
                               const int* __restrict__ seq_of_row, const int* __restrict__ row_start,
                               const int* __restrict__ seq_begin, const int* __restrict__ state_slots,
                               const int* __restrict__ block_table, int bt_stride, const float* __restrict__ inv_freq,
                               ConvGeometry g, int write_kv, int rows) {
    constexpr int N = Packet<T>::N;
    constexpr int ROWS = SINGLE ? 1 : kRowTile;      // (a step of single rows has few of them: a thread a row)
    pdl_trigger();
    pdl_wait();                                   // the projected rows and the step's metadata come from kernels in front
    const int packet = blockIdx.y * blockDim.x + threadIdx.x;
    if (packet >= g.channels / N) return;
    const int c0 = packet * N;
    int segment, head, e0;
    if (c0 < g.heads * g.dim) {
        segment = 0; head = c0 / g.dim; e0 = c0 % g.dim;
    } else if (c0 < (g.heads + g.kv_heads) * g.dim) {
        segment = 1; head = (c0 - g.heads * g.dim) / g.dim; e0 = (c0 - g.heads * g.dim) % g.dim;
    } else {
        const int local = c0 - (g.heads + g.kv_heads) * g.dim;
        segment = 2; head = local / g.vdim; e0 = local % g.vdim;
    }
    float w[J][N];                                   // the packet's taps: neighbouring lanes read neighbouring packets
#pragma unroll
    for (int j = 0; j < J; ++j) load_floats<N>(taps + (int64_t)j * g.channels + c0, w[j]);
    const bool rotates = segment < 2 && e0 < g.rot_dims;
    const int64_t page_elems = (int64_t)g.kv_heads * g.page_size * (g.dim + g.vdim);

    // what the rows of the tile are, asked for at once (each is a chain of two or three dependent loads)
    int row_pos[ROWS], row_begin[ROWS], row_first[ROWS], row_slot[ROWS], row_page[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int row = min(blockIdx.x * ROWS + r, rows - 1);
        const int seq = seq_of_row[row];
        row_pos[r] = positions[row];
        row_begin[r] = seq_begin[seq];
        row_first[r] = row_start[seq];
        row_slot[r] = state_slots[seq];
        row_page[r] = (segment != 0 && write_kv) ? block_table[(int64_t)seq * bt_stride + row_pos[r] / g.page_size] : 0;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const int row = blockIdx.x * ROWS + r;
        if (row >= rows) return;
        const int pos = row_pos[r];
        const int begin = row_begin[r];
        const int first_row = row_first[r];
        float* st = state + (int64_t)row_slot[r] * (J - 1) * g.channels + c0;
        float u[J][N];
#pragma unroll
        for (int j = 0; j < J; ++j) {
            const int p = pos - (J - 1) + j;
            if (p >= begin) {
                Packet<T>::load(proj + (int64_t)(first_row + (p - begin)) * proj_stride + c0, u[j]);
            } else if (p >= 0) {
                load_floats<N>(st + (int64_t)(p - (begin - (J - 1))) * g.channels, u[j]);
            } else {
#pragma unroll
                for (int e = 0; e < N; ++e) u[j][e] = 0.0f;
            }
        }
        float y[N];
#pragma unroll
        for (int e = 0; e < N; ++e) {
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < J; ++j) sum = fmaf(w[j][e], u[j][e], sum);
            y[e] = sum;
        }
        if (SINGLE) {
#pragma unroll
            for (int j = 1; j < J; ++j) store_floats<N>(st + (int64_t)(j - 1) * g.channels, u[j]);
        }
        if (rotates) {
#pragma unroll
            for (int e = 0; e < N; e += 2) {
                if (e0 + e < g.rot_dims) {
                    float sn, cs;
                    sincosf((float)pos * inv_freq[(e0 + e) >> 1], &sn, &cs);
                    const float r0 = y[e] * cs - y[e + 1] * sn;
                    const float r1 = y[e + 1] * cs + y[e] * sn;
                    y[e] = r0;
                    y[e + 1] = r1;
                }
            }
        }
        if (segment == 0) {
            Packet<T>::store(q_out + (int64_t)row * q_stride + c0, y);
        } else if (write_kv) {
            const int in_page = pos % g.page_size;
            T* dst = cache + (int64_t)row_page[r] * page_elems;
            if (segment == 1) dst += ((int64_t)head * g.page_size + in_page) * g.dim + e0;
            else dst += (int64_t)g.kv_heads * g.page_size * g.dim + ((int64_t)head * g.page_size + in_page) * g.vdim + e0;
            Packet<T>::store(dst, y);
        }
    }
}

// New state of every sequence of the step: index i holds the projected row of position begin + n - (J - 1) + i,
// which is a row of this step, an older row of the state, or zero (before the sequence's start).  One thread owns
// a channel of a sequence, reads all it needs and only then writes.
template <typename T>
__global__ void conv_state_update_kernel(const T* __restrict__ proj, int64_t proj_stride, float* __restrict__ state,
                                         const int* __restrict__ row_start, const int* __restrict__ seq_begin,
                                         const int* __restrict__ state_slots, int channels, int J) {
    pdl_trigger();
    pdl_wait();                                   // the convolution in front still reads the old state
    const int seq = blockIdx.x;
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int first_row = row_start[seq];
    const int n = row_start[seq + 1] - first_row;
    const int begin = seq_begin[seq];
    float* st = state + (int64_t)state_slots[seq] * (J - 1) * channels + c;
    float fresh[kMaxTaps];
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i) {
        if (i < J - 1) {
            const int p = begin + n - (J - 1) + i;
            float v = 0.0f;
            if (p >= begin) v = Elem<T>::load(proj + (int64_t)(first_row + (p - begin)) * proj_stride + c);
            else if (p >= 0) v = st[(int64_t)(p - (begin - (J - 1))) * channels];
            fresh[i] = v;
        }
    }
#pragma unroll
    for (int i = 0; i < kMaxTaps - 1; ++i)
        if (i < J - 1) st[(int64_t)i * channels] = fresh[i];
}

ConvGeometry geometry(int heads, int kv_heads, int dim, int vdim, int rot_dims, int taps, int page_size) {
    ConvGeometry g;
    g.heads = heads; g.kv_heads = kv_heads; g.dim = dim; g.vdim = vdim; g.rot_dims = rot_dims; g.taps = taps;
    g.page_size = page_size;
    g.channels = heads * dim + kv_heads * dim + kv_heads * vdim;
    g.q_pairs = heads * ((dim + 1) / 2);
    g.k_pairs = kv_heads * ((dim + 1) / 2);
    g.v_pairs = kv_heads * ((vdim + 1) / 2);
    return g;
}

template <typename T>
int launch(const void* proj, int64_t proj_stride, const float* taps, float* state, void* q_out, int64_t q_stride,
           void* cache, const int* positions, const int* seq_of_row, const int* row_start, const int* seq_begin,
           const int* state_slots, const int* block_table, int bt_stride, const float* inv_freq, int rows,
           const ConvGeometry& g, int write_kv, int single, cudaStream_t stream) {
    constexpr int N = Packet<T>::N;
    const uintptr_t bits = (uintptr_t)proj | (uintptr_t)q_out | (uintptr_t)cache | (uintptr_t)state | (uintptr_t)taps;
    if (g.dim % N == 0 && g.vdim % N == 0 && g.taps <= 4 && proj_stride % N == 0 && q_stride % N == 0 &&
        bits % 16 == 0) {
        const int tile = single ? 1 : kRowTile;
        const dim3 tiles((rows + tile - 1) / tile, (g.channels / N + 127) / 128);
#define TB_CONV(S, J)                                                                                             \
    tb_launch_pdl(conv_rope_cache_packets_kernel<T, S, J>, tiles, dim3(128), 0, stream, (const T*)proj,           \
                  proj_stride, taps, state, (T*)q_out, q_stride, (T*)cache, positions, seq_of_row, row_start,     \
                  seq_begin, state_slots, block_table, bt_stride, inv_freq, g, write_kv, rows)
        if (single) {
            if (g.taps == 1) TB_CONV(true, 1); else if (g.taps == 2) TB_CONV(true, 2);
            else if (g.taps == 3) TB_CONV(true, 3); else TB_CONV(true, 4);
        } else {
            if (g.taps == 1) TB_CONV(false, 1); else if (g.taps == 2) TB_CONV(false, 2);
            else if (g.taps == 3) TB_CONV(false, 3); else TB_CONV(false, 4);
        }
#undef TB_CONV
        return tb_launch_status();
    }
    const int total = g.q_pairs + g.k_pairs + g.v_pairs;
    const dim3 grid(rows, (total + 127) / 128);
    if (single)
        tb_launch_pdl(conv_rope_cache_kernel<T, true>, grid, dim3(128), 0, stream, (const T*)proj, proj_stride, taps,
                      state, (T*)q_out, q_stride, (T*)cache, positions, seq_of_row, row_start, seq_begin, state_slots,
                      block_table, bt_stride, inv_freq, g, write_kv);
    else
        tb_launch_pdl(conv_rope_cache_kernel<T, false>, grid, dim3(128), 0, stream, (const T*)proj, proj_stride, taps,
                      state, (T*)q_out, q_stride, (T*)cache, positions, seq_of_row, row_start, seq_begin, state_slots,
                      block_table, bt_stride, inv_freq, g, write_kv);
    return tb_launch_status();
}

}  // namespace

// proj: [rows, >= channels] with row stride proj_stride (elements); taps: 32-bit [taps, channels] (tap j of
// every channel side by side: tap taps - 1 multiplies the row itself, tap 0 the oldest);
// state: 32-bit [slots, taps - 1, channels]; q_out: [rows, heads * dim] with row stride q_stride;
// cache: this layer's pages; inv_freq: 32-bit [rot_dims / 2] (may be null when rot_dims is 0).
// single != 0: every sequence of the step brings exactly one row, and the state is renewed here.
TB_EXPORT int tb_conv_rope_cache(const void* proj, int64_t proj_stride, const float* taps, float* state, void* q_out,
                                 int64_t q_stride, void* cache, const int* positions, const int* seq_of_row,
                                 const int* row_start, const int* seq_begin, const int* state_slots,
                                 const int* block_table, int bt_stride, const float* inv_freq, int rows, int heads,
                                 int kv_heads, int dim, int vdim, int rot_dims, int taps_count, int page_size,
                                 int write_kv, int single, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (taps_count < 1 || taps_count > kMaxTaps) return TB_ERR_BAD_SIZE;
    if (heads < 1 || kv_heads < 1 || dim < 1 || vdim < 1 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (rot_dims < 0 || rot_dims > dim || rot_dims % 2 != 0) return TB_ERR_BAD_SIZE;
    const ConvGeometry g = geometry(heads, kv_heads, dim, vdim, rot_dims, taps_count, page_size);
    if (dtype == TB_F32)
        return launch<float>(proj, proj_stride, taps, state, q_out, q_stride, cache, positions, seq_of_row, row_start,
                             seq_begin, state_slots, block_table, bt_stride, inv_freq, rows, g, write_kv, single, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(proj, proj_stride, taps, state, q_out, q_stride, cache, positions, seq_of_row,
                                     row_start, seq_begin, state_slots, block_table, bt_stride, inv_freq, rows, g,
                                     write_kv, single, stream);
    return TB_ERR_BAD_DTYPE;
}

TB_EXPORT int tb_conv_state_update(const void* proj, int64_t proj_stride, float* state, const int* row_start,
                                   const int* seq_begin, const int* state_slots, int num_seqs, int channels,
                                   int taps_count, int dtype, cudaStream_t stream) {
    if (num_seqs == 0 || taps_count <= 1) return 0;
    if (taps_count > kMaxTaps) return TB_ERR_BAD_SIZE;
    const dim3 grid(num_seqs, (channels + 127) / 128);
    if (dtype == TB_F32)
        tb_launch_pdl(conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, proj_stride, state,
                      row_start, seq_begin, state_slots, channels, taps_count);
    else if (dtype == TB_BF16)
        tb_launch_pdl(conv_state_update_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, (const __nv_bfloat16*)proj,
                      proj_stride, state, row_start, seq_begin, state_slots, channels, taps_count);
    else
        return TB_ERR_BAD_DTYPE;
    return tb_launch_status();
}
