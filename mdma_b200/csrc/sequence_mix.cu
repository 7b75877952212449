// Kernels of layers that carry fixed-size state from token to token, and of the small
// element-wise steps around them: a norm without statistics (dynamic tanh), the
// token shift, the gated residual add, a gated linear recurrence (minGRU), a short causal
// convolution, the selective state-space scan (Mamba-2) with its gated group norm, the
// soft cap of the logits.  Templates over the activation type (float in the 32-bit
// engine, bfloat16 in the serving engine) and over the type the small vectors are kept
// in.  Everything that enters a recurrence, the state itself, the norms and the residual
// sum are float in both engines.
//
// The step's tokens are a flat batch: sequence s of the step owns rows
// [seq_start[s], seq_start[s+1]) and keeps its state in row seq_slot[s] of a state
// tensor whose rows are `state_stride` floats apart.  A kernel that reads a sequence's
// state for the first row and a kernel that writes it from the last row are never the
// same launch unless one thread does both, so a step of many rows and a step of one
// row leave the same state.
#include "common.cuh"

namespace mdma {

// Row-wise kernels run a grid of (rows, column parts): a step of a few rows still fills the device, and no
// thread walks a row with one dependent load after another.
static inline unsigned column_parts(int width) {
    const int parts = (width + 255) / 256;
    return (unsigned)(parts < 1 ? 1 : parts > 64 ? 64 : parts);
}

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// Row kernels take VEC = 4 consecutive columns a thread (16-byte accesses of the float rows, 8-byte ones of
// bfloat16 rows) when the width and every row pitch are multiples of 4, else one.
template <int VEC, typename T> struct RowVec;
template <typename T> struct RowVec<1, T> {
    static __device__ __forceinline__ void load(const T* p, float* v) { v[0] = to_float(p[0]); }
    static __device__ __forceinline__ void store(T* p, const float* v) { p[0] = from_float<T>(v[0]); }
};
template <> struct RowVec<4, float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        const float4 q = *reinterpret_cast<const float4*>(p);
        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct RowVec<4, __nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        const uint2 q = *reinterpret_cast<const uint2*>(p);
        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
        v[0] = lo.x; v[1] = lo.y; v[2] = hi.x; v[3] = hi.y;
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 q;
        q.x = *reinterpret_cast<uint32_t*>(&lo); q.y = *reinterpret_cast<uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = q;
    }
};
#define MDMA_ROW_LOOP(e, width, VEC) \
    for (int e = (blockIdx.y * blockDim.x + threadIdx.x) * VEC; e < width; e += gridDim.y * blockDim.x * VEC)

// ---------------------------------------------------------------- dynamic tanh
// y[r,:] = tanh(alpha * x[src,:]) * w + b, src = rows[r] or r.  No sum over the row.
template <typename TO, typename TW, int VEC>
__global__ void __launch_bounds__(256)
dyt_norm_kernel(const float* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                const TW* __restrict__ alpha, const int* __restrict__ rows, TO* __restrict__ y, int width) {
    chain_release();
    chain_wait();
    const int r = blockIdx.x;
    const float a = to_float(alpha[0]);
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    TO* yr = y + (size_t)r * width;
    MDMA_ROW_LOOP(e, width, VEC) {
        float xv[VEC], wv[VEC], bv[VEC], out[VEC];
        RowVec<VEC, float>::load(xr + e, xv);
        RowVec<VEC, TW>::load(w + e, wv);
        RowVec<VEC, TW>::load(b + e, bv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) out[i] = tanhf(a * xv[i]) * wv[i] + bv[i];
        RowVec<VEC, TO>::store(yr + e, out);
    }
}

// The same with the token shift behind it: h = dyt(x[t]) and hs = h + (h' - h) * mu, h' the h of the
// row before in the same sequence (recomputed from x, which costs nothing for a norm without sums) or,
// for a sequence's first row of the step, the kept one.  Both h and h' are rounded to the activation
// type first, so that the kept value and the recomputed one are the same number.
template <typename TO, typename TW, int VEC>
__global__ void __launch_bounds__(256)
dyt_shift_kernel(const float* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                 const TW* __restrict__ alpha, const TW* __restrict__ mu, const int* __restrict__ tok_seq,
                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                 const float* __restrict__ state, long state_stride, TO* __restrict__ h, TO* __restrict__ hs, int width) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int s = tok_seq[t];
    const bool first = t == seq_start[s];
    const float a = to_float(alpha[0]);
    const float* xr = x + (size_t)t * width;
    const float* prev = first ? state + (size_t)seq_slot[s] * state_stride : xr - width;
    MDMA_ROW_LOOP(e, width, VEC) {
        float xv[VEC], pv[VEC], wv[VEC], bv[VEC], mv[VEC], cur[VEC], shifted[VEC];
        RowVec<VEC, float>::load(xr + e, xv);
        RowVec<VEC, float>::load(prev + e, pv);
        RowVec<VEC, TW>::load(w + e, wv);
        RowVec<VEC, TW>::load(b + e, bv);
        RowVec<VEC, TW>::load(mu + e, mv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            cur[i] = to_float(from_float<TO>(tanhf(a * xv[i]) * wv[i] + bv[i]));
            const float before = first ? pv[i] : to_float(from_float<TO>(tanhf(a * pv[i]) * wv[i] + bv[i]));
            shifted[i] = cur[i] + (before - cur[i]) * mv[i];
        }
        RowVec<VEC, TO>::store(h + (size_t)t * width + e, cur);
        RowVec<VEC, TO>::store(hs + (size_t)t * width + e, shifted);
    }
}

// ---------------------------------------------------------------- token shift
// hs[t] = h[t] + (h' - h[t]) * mu, h' = h[t-1] inside the step, the kept row at its start.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
token_shift_kernel(const T* __restrict__ h, const TW* __restrict__ mu, const int* __restrict__ tok_seq,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                   const float* __restrict__ state, long state_stride, T* __restrict__ hs, int width) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int s = tok_seq[t];
    const bool first = t == seq_start[s];
    const T* cur = h + (size_t)t * width;
    const float* kept = state + (size_t)seq_slot[s] * state_stride;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x) {
        const float c = to_float(cur[e]);
        const float before = first ? kept[e] : to_float(cur[e - width]);
        hs[(size_t)t * width + e] = from_float<T>(c + (before - c) * to_float(mu[e]));
    }
}

// state[slot of s] = float(rows[last row of s]): what the next step's first row reads.
template <typename T>
__global__ void __launch_bounds__(256)
keep_last_rows_kernel(const T* __restrict__ rows, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                      float* __restrict__ state, long state_stride, int width) {
    chain_release();
    chain_wait();
    const int s = blockIdx.x;
    const T* last = rows + (size_t)(seq_start[s + 1] - 1) * width;
    float* kept = state + (size_t)seq_slot[s] * state_stride;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x) kept[e] = to_float(last[e]);
}

// ---------------------------------------------------------------- gated residual add
// x[t,:] += sigmoid(g[t,:]) * y[t,:].  With `keep_rows` the rows of it that end a sequence go to
// the state as well (the token shift's kept row), which saves a launch.  With `splits` > 0, y is the sum of
// that many partial results [split][row][width] (a K-split product whose reduction is done here).
template <typename TG, typename TK, int VEC>
__global__ void __launch_bounds__(256)
gated_add_kernel(float* __restrict__ x, const TG* __restrict__ g, const float* __restrict__ y,
                 const float* __restrict__ partial, int splits, size_t split_stride, int width,
                 const TK* __restrict__ keep_rows, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                 const int* __restrict__ seq_slot, float* __restrict__ state, long state_stride) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const size_t o = (size_t)t * width;
    MDMA_ROW_LOOP(e, width, VEC) {
        // y is either complete or still the K-split partial sums of the product that made it, added up here in split order
        float v[VEC], xv[VEC], gv[VEC];
        if (splits > 0) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) v[i] = 0.f;
            for (int sp = 0; sp < splits; ++sp) {
                float pv[VEC];
                RowVec<VEC, float>::load(partial + (size_t)sp * split_stride + o + e, pv);
#pragma unroll
                for (int i = 0; i < VEC; ++i) v[i] += pv[i];
            }
        } else {
            RowVec<VEC, float>::load(y + o + e, v);
        }
        RowVec<VEC, float>::load(x + o + e, xv);
        RowVec<VEC, TG>::load(g + o + e, gv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) xv[i] = xv[i] + sigmoid_f(gv[i]) * v[i];
        RowVec<VEC, float>::store(x + o + e, xv);
    }
    if (keep_rows != nullptr) {
        const int s = tok_seq[t];
        if (t == seq_start[s + 1] - 1) {
            float* kept = state + (size_t)seq_slot[s] * state_stride;
            MDMA_ROW_LOOP(e, width, VEC) {
                float kv[VEC];
                RowVec<VEC, TK>::load(keep_rows + o + e, kv);
                RowVec<VEC, float>::store(kept + e, kv);
            }
        }
    }
}

// ---------------------------------------------------------------- activation, soft cap, row packing
template <typename T>
__global__ void activation_kernel(T* __restrict__ v, long n, int act) {
    chain_release();
    chain_wait();
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        v[i] = from_float<T>(gate_activation(to_float(v[i]), act));
}

// v = cap * tanh(v / cap): logits bounded to (-cap, cap).
__global__ void softcap_kernel(float* __restrict__ v, long n, float cap) {
    chain_release();
    chain_wait();
    const float inv = 1.0f / cap;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        v[i] = cap * tanhf(v[i] * inv);
}

// out[t,:] = [a[t,:] | b[t,:]] in the activation type: the operand of a product over two float streams.
template <typename T>
__global__ void __launch_bounds__(256)
pack_pair_kernel(const float* __restrict__ a, const float* __restrict__ b, T* __restrict__ out, int width) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x) {
        out[(size_t)t * 2 * width + e] = from_float<T>(a[(size_t)t * width + e]);
        out[(size_t)t * 2 * width + width + e] = from_float<T>(b[(size_t)t * width + e]);
    }
}

// ---------------------------------------------------------------- minGRU
// p[t] = [pz | pu | pg] (three projections of `width` columns, float).  z = sigmoid(pz + bz),
// u = pu + bu, candidate = u + 1/2 (u >= 0) or sigmoid(u) (u < 0); S = (1 - z) S + z candidate;
// out = S * silu(pg).  One thread per (sequence, channel) walks the step's rows in order.
template <typename TO, typename TW>
__global__ void __launch_bounds__(128)
mingru_scan_kernel(const float* __restrict__ p, int p_stride, const TW* __restrict__ bz, const TW* __restrict__ bu,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ state,
                   long state_stride, TO* __restrict__ out, int width) {
    chain_release();
    chain_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= width) return;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    float* kept = state + (size_t)seq_slot[s] * state_stride + c;
    float S = *kept;
    const float zb = to_float(bz[c]), ub = to_float(bu[c]);
    for (int t = t0; t < t1; ++t) {
        const float* row = p + (size_t)t * p_stride;
        const float z = sigmoid_f(row[c] + zb);
        const float u = row[width + c] + ub;
        const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
        S = (1.0f - z) * S + z * cand;
        out[(size_t)t * width + c] = from_float<TO>(S * silu_f(row[2 * width + c]));
    }
    *kept = S;
}

// The same recurrence for steps that bring many rows per sequence: it is linear in S (S_t = a_t S_(t-1) + b_t with
// a = 1 - z, b = z * candidate), so a sequence's rows are cut into kGruChunks (128) runs; a thread walks one run of one
// channel from zero and keeps the run's product of a and its last value, the runs' starting values follow from
// those in order, and every run is walked again from its starting value, this time writing the outputs.  The
// association of the products differs from the row-by-row kernel's, so results agree to rounding, not to the bit:
// the serving engine uses this kernel, the 32-bit engine the one above.
// eight channels are one 32-byte sector of a row: narrow blocks, so that one sequence already gives width / 8 of them
constexpr int kGruChunks = 128, kGruChannels = 8;

template <typename TO, typename TW>
__global__ void __launch_bounds__(kGruChunks * kGruChannels)
mingru_scan_chunked_kernel(const float* __restrict__ p, int p_stride, const TW* __restrict__ bz, const TW* __restrict__ bu,
                           const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ state,
                           long state_stride, TO* __restrict__ out, int width) {
    chain_release();
    chain_wait();
    __shared__ float sA[kGruChunks][kGruChannels], sB[kGruChunks][kGruChannels];
    const int lane_c = threadIdx.x % kGruChannels, k = threadIdx.x / kGruChannels;
    const int c = blockIdx.x * kGruChannels + lane_c;
    const int s = blockIdx.y;
    const bool live = c < width;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    const int run = (t1 - t0 + kGruChunks - 1) / kGruChunks;
    const int lo = min(t1, t0 + k * run), hi = min(t1, lo + run);
    const float zb = live ? to_float(bz[c]) : 0.f, ub = live ? to_float(bu[c]) : 0.f;
    float A = 1.f, B = 0.f;
    if (live) {
        for (int t = lo; t < hi; ++t) {
            const float* row = p + (size_t)t * p_stride;
            const float z = sigmoid_f(row[c] + zb);
            const float u = row[width + c] + ub;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            A *= 1.0f - z;
            B = (1.0f - z) * B + z * cand;
        }
    }
    sA[k][lane_c] = A;
    sB[k][lane_c] = B;
    __syncthreads();
    if (k == 0 && live) {
        float* kept = state + (size_t)seq_slot[s] * state_stride + c;
        float S = *kept;
        for (int j = 0; j < kGruChunks; ++j) {
            const float next = sA[j][lane_c] * S + sB[j][lane_c];
            sB[j][lane_c] = S;                       // the run's starting value
            S = next;
        }
        *kept = S;
    }
    __syncthreads();
    if (live) {
        float S = sB[k][lane_c];
        for (int t = lo; t < hi; ++t) {
            const float* row = p + (size_t)t * p_stride;
            const float z = sigmoid_f(row[c] + zb);
            const float u = row[width + c] + ub;
            const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
            S = (1.0f - z) * S + z * cand;
            out[(size_t)t * width + c] = from_float<TO>(S * silu_f(row[2 * width + c]));
        }
    }
}

// ---------------------------------------------------------------- short causal convolution
// out[t,c] = silu(sum_j w[c,j] * in(t - (taps-1) + j, c) + b[c]) (or the sum itself, `silu` = 0); in(.) is column in_col + c of the
// projection rows of this step, or, before the step's first row of the sequence, the kept inputs
// (`state`: [taps-1, channels] floats per slot, oldest first; zeros before the sequence's start).
template <typename TW, typename TB, int VEC>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const float* __restrict__ proj, int proj_stride, int in_col, const TW* __restrict__ w,
                        const TB* __restrict__ b, int taps, int channels, const int* __restrict__ tok_seq,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                        const float* __restrict__ state, long state_stride, float* __restrict__ out, int silu) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int s = tok_seq[t];
    const int t0 = seq_start[s];
    const float* kept = state + (size_t)seq_slot[s] * state_stride;
    MDMA_ROW_LOOP(c, channels, VEC) {
        float acc[VEC];
        RowVec<VEC, TB>::load(b + c, acc);
        for (int j = 0; j < taps; ++j) {
            const int src = t - (taps - 1) + j;            // a row of this step, or before it
            float v[VEC];
            RowVec<VEC, float>::load(src >= t0 ? proj + (size_t)src * proj_stride + in_col + c
                                               : kept + (size_t)(taps - 1 + (src - t0)) * channels + c, v);
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = fmaf(to_float(w[(size_t)(c + i) * taps + j]), v[i], acc[i]);
        }
        if (silu) {
#pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] = silu_f(acc[i]);
        }
        RowVec<VEC, float>::store(out + (size_t)t * channels + c, acc);
    }
}

// The kept inputs after the step: the last taps-1 inputs of the sequence, from this step's rows and,
// if it brought fewer, from what was kept before.  One thread per (sequence, channel) reads all it
// needs before it writes.
constexpr int kMaxTaps = 16;
__global__ void __launch_bounds__(256)
conv_keep_kernel(const float* __restrict__ proj, int proj_stride, int in_col, int taps, int channels,
                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ state,
                 long state_stride) {
    chain_release();
    chain_wait();
    const int s = blockIdx.y;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    float* kept = state + (size_t)seq_slot[s] * state_stride;
    float v[kMaxTaps];
    const int keep = taps - 1;
    for (int j = 0; j < keep; ++j) {
        const int src = t1 - keep + j;
        v[j] = src >= t0 ? proj[(size_t)src * proj_stride + in_col + c] : kept[(size_t)(keep + (src - t0)) * channels + c];
    }
    for (int j = 0; j < keep; ++j) kept[(size_t)j * channels + c] = v[j];
}

// ---------------------------------------------------------------- Mamba-2 scan
// Per head h (group g = h / (heads / groups)), token by token:
//   dt = softplus(raw + dt_bias[h]);  S = exp(-exp(A_log[h]) dt) S + dt B x^T  (S: [N, vdim]);
//   y = S^T C + D[h] x.
// `conv` rows hold [x: heads*vdim | B: groups*N | C: groups*N] after the convolution, `proj` rows the
// raw dt at column dt_col + h.  A block owns VB value columns of one (sequence, head); NP lanes share a
// column, each with NPER of the N state rows in registers; the step's rows are staged through shared
// memory sixteen at a time.  The state of a (sequence, head, column) is read and written by the same threads;
// it is kept as [head][column][N], so that the lanes that share a column touch neighbouring words.
//
// Steps that bring many rows per sequence cut every sequence into runs of `chunk_rows` rows that are walked side
// by side (the recurrence is linear in S): pass kScanLocal walks each run but the last from S = 0 and leaves the
// run's last S and its total decay exp(-exp(A_log) sum dt) in scratch; mamba2_chunk_starts_kernel turns those, in
// order, into every run's starting S; pass kScanFrom walks every run from its starting S and writes y (the last run
// writes the sequence's state).  Twice the arithmetic for as many times the blocks; equal to the one-pass walk up
// to rounding, so the serving engine uses it and the 32-bit engine does not.
constexpr int kScanRows = 16;
enum ScanPass : int { kScanWhole = 0, kScanLocal = 1, kScanFrom = 2 };

// NPT: the lanes that share a value column, when known at compile time (the common state sizes: loops unroll and
// the index arithmetic folds), or 0: the run-time value `np_lanes` is used.
// TS: the type of the state, of the step sizes and decays and of the sums over the state: float, or double in the
// exact engine (a decay is a product of up to thousands of factors below one, each rounded; in float that chain of
// roundings, not the matrix products, is what a long sequence's result differs by from the exact one).  A double
// state occupies two of the state row's floats per element.
// 4-byte copies from global to shared memory that do not hold the thread up (cp.async), in groups that are waited for.
__device__ __forceinline__ void async_copy_4(float* dst_shared, const float* src_global) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(dst_shared);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"(d), "l"(src_global) : "memory");
}
__device__ __forceinline__ void async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <typename TS> __device__ __forceinline__ TS exp_t(TS v);
template <> __device__ __forceinline__ float exp_t<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double exp_t<double>(double v) { return exp(v); }
template <typename TS> __device__ __forceinline__ TS softplus_t(TS v);
template <> __device__ __forceinline__ float softplus_t<float>(float v) { return softplus_f(v); }
template <> __device__ __forceinline__ double softplus_t<double>(double v) { return v > 40.0 ? v : log1p(exp(v)); }

template <int NPER, int VPT, int NPT, typename TW, int PASS, typename TS = float>
__global__ void __launch_bounds__(128)
mamba2_scan_kernel(const float* __restrict__ conv, int conv_stride, const float* __restrict__ proj, int proj_stride,
                   int dt_col, const TW* __restrict__ dt_bias, const TW* __restrict__ A_log, const TW* __restrict__ D,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ state,
                   long state_stride, float* __restrict__ y, int heads, int vdim, int N, int G, int np_lanes,
                   int chunk_rows, int max_chunks, float* __restrict__ chunk_state, float* __restrict__ chunk_decay) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float sm[];
    const int NP = NPT > 0 ? NPT : np_lanes;
    // a thread owns NPER state rows of VPT value columns: B and C, which every column needs, are fetched once for
    // VB = (threads / NP) * VPT columns
    const int VB = blockDim.x / NP * VPT;
    const int Npad = NP * NPER;
    // The rows are staged through two sets of buffers: while one set of 16 rows is walked, the next is on its way
    // (cp.async), so that the walk never waits for global memory.
    TS* sdt = reinterpret_cast<TS*>(sm);                          // first: doubles want 8-byte alignment
    TS* sa = sdt + kScanRows;
    float* stage0 = reinterpret_cast<float*>(sa + kScanRows);
    const int s = PASS == kScanWhole ? blockIdx.x : blockIdx.x / max_chunks;
    const int run = PASS == kScanWhole ? 0 : blockIdx.x % max_chunks;
    const int h = blockIdx.y, v0 = blockIdx.z * VB;
    const int inner_cols = heads * vdim, g_col = (h / (heads / G)) * N;
    int t_begin = seq_start[s], t_end = seq_start[s + 1];
    bool last_run = true;
    if (PASS != kScanWhole) {
        const int runs = (t_end - t_begin + chunk_rows - 1) / chunk_rows;
        last_run = run == runs - 1;
        if (run >= runs || (PASS == kScanLocal && last_run)) return;       // the whole block leaves together
        t_begin += run * chunk_rows;
        t_end = min(t_end, t_begin + chunk_rows);
    }
    const size_t state_floats = (size_t)heads * N * vdim;
    const int np = threadIdx.x % NP, vl = (threadIdx.x / NP) * VPT;       // first of this thread's columns, within the block
    const int inner = heads * vdim;
    TS* Sg = reinterpret_cast<TS*>(state + (size_t)seq_slot[s] * state_stride) + (size_t)h * N * vdim;
    TS* Sc = PASS == kScanWhole ? nullptr
                                : reinterpret_cast<TS*>(chunk_state) + (size_t)blockIdx.x * state_floats + (size_t)h * N * vdim;
    const TS* Sfrom = PASS == kScanWhole ? Sg : Sc;
    TS S[VPT][NPER];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        const int v = v0 + vl + j;
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
            const int n = np * NPER + i;
            S[j][i] = (PASS != kScanLocal && v < vdim && n < N) ? Sfrom[(size_t)v * N + n] : TS(0);
        }
    }
    TS dt_sum = 0;
    const TS rate = exp_t<TS>((TS)to_float(A_log[h])), bias = (TS)to_float(dt_bias[h]);
    const float Dh = to_float(D[h]);
    const int stage_floats = kScanRows * (2 * Npad + VB + 1);     // B, C, x and the raw step sizes of 16 rows
    auto issue = [&](int t0, int nt, float* base) {
        float* pB = base; float* pC = pB + kScanRows * Npad; float* px = pC + kScanRows * Npad; float* pr = px + kScanRows * VB;
        for (int i = threadIdx.x; i < nt * Npad; i += blockDim.x) {
            const int tt = i / Npad, n = i % Npad;
            if (n < N) {
                const float* row = conv + (size_t)(t0 + tt) * conv_stride + inner_cols + g_col;
                async_copy_4(pB + i, row + n);
                if (PASS != kScanLocal) async_copy_4(pC + i, row + G * N + n);
            }
        }
        for (int i = threadIdx.x; i < nt * VB; i += blockDim.x) {
            const int tt = i / VB, vv = i % VB;
            if (v0 + vv < vdim) async_copy_4(px + i, conv + (size_t)(t0 + tt) * conv_stride + h * vdim + v0 + vv);
        }
        for (int i = threadIdx.x; i < nt; i += blockDim.x)
            async_copy_4(pr + i, proj + (size_t)(t0 + i) * proj_stride + dt_col + h);
        async_commit();
    };
    // entries that no copy writes (state rows beyond N, value columns beyond vdim), if there are any, are zero in both sets
    if (Npad > N || v0 + VB > vdim) {
        for (int i = threadIdx.x; i < 2 * stage_floats; i += blockDim.x) stage0[i] = 0.f;
        __syncthreads();
    }
    int set = 0;
    if (t_begin < t_end) issue(t_begin, min(kScanRows, t_end - t_begin), stage0);
    for (int t0 = t_begin; t0 < t_end; t0 += kScanRows, set ^= 1) {
        const int nt = min(kScanRows, t_end - t0);
        float* base = stage0 + set * stage_floats;
        const float* sB = base;
        const float* sC = sB + kScanRows * Npad;
        const float* sx = sC + kScanRows * Npad;
        const float* sraw = sx + kScanRows * VB;
        // the other set was read in the round before (the barrier at this loop's end): fill it with the next rows
        if (t0 + kScanRows < t_end) {
            issue(t0 + kScanRows, min(kScanRows, t_end - t0 - kScanRows), stage0 + (set ^ 1) * stage_floats);
            async_wait_but_one();
        } else {
            async_wait_all();
        }
        __syncthreads();                                   // this set's rows have landed, for every thread
        for (int i = threadIdx.x; i < nt; i += blockDim.x) {
            const TS d = softplus_t<TS>((TS)sraw[i] + bias);
            sdt[i] = d;
            sa[i] = exp_t<TS>(-rate * d);
        }
        __syncthreads();
        if (PASS == kScanLocal && threadIdx.x == 0)
            for (int tt = 0; tt < nt; ++tt) dt_sum += sdt[tt];
        for (int tt = 0; tt < nt; ++tt) {
            const TS a = sa[tt], dt = sdt[tt];
            // a thread's NPER entries of B and of C lie side by side: 16-byte shared-memory loads
            float Bt[NPER], Ct[NPER];
#pragma unroll
            for (int i = 0; i < NPER; i += 4) {
                const float4 b4 = *reinterpret_cast<const float4*>(sB + tt * Npad + np * NPER + i);
                Bt[i] = b4.x; Bt[i + 1] = b4.y; Bt[i + 2] = b4.z; Bt[i + 3] = b4.w;
                if (PASS != kScanLocal) {
                    const float4 c4 = *reinterpret_cast<const float4*>(sC + tt * Npad + np * NPER + i);
                    Ct[i] = c4.x; Ct[i + 1] = c4.y; Ct[i + 2] = c4.z; Ct[i + 3] = c4.w;
                }
            }
            TS acc[VPT];
            float xv[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                xv[j] = sx[tt * VB + vl + j];
                const TS dtx = dt * (TS)xv[j];
                acc[j] = 0;
#pragma unroll
                for (int i = 0; i < NPER; ++i) {
                    S[j][i] = a * S[j][i] + dtx * (TS)Bt[i];              // one fused multiply-add and a multiply
                    if (PASS != kScanLocal) acc[j] += S[j][i] * (TS)Ct[i];
                }
            }
            if (PASS != kScanLocal) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
#pragma unroll
                    for (int o = NP >> 1; o > 0; o >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
                    const int v = v0 + vl + j;
                    if (np == 0 && v < vdim) y[(size_t)(t0 + tt) * inner + h * vdim + v] = (float)(acc[j] + (TS)Dh * (TS)xv[j]);
                }
            }
        }
        __syncthreads();                                   // everyone is done with this set and with sdt, sa
    }
    TS* Sto = PASS == kScanLocal ? Sc : (last_run ? Sg : nullptr);
    if (Sto != nullptr) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int v = v0 + vl + j;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                const int n = np * NPER + i;
                if (v < vdim && n < N) Sto[(size_t)v * N + n] = S[j][i];
            }
        }
    }
    if (PASS == kScanLocal && threadIdx.x == 0 && blockIdx.z == 0)
        chunk_decay[(size_t)blockIdx.x * heads + h] = (float)exp_t<TS>(-rate * dt_sum);
}

// The runs' starting states, in order: start[0] = the sequence's state, start[r+1] = decay[r] * start[r] + local[r].
// `chunk_state` holds local[r] on entry and start[r] on return.  One thread per state element.
__global__ void __launch_bounds__(256)
mamba2_chunk_starts_kernel(const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                           const float* __restrict__ state, long state_stride, float* __restrict__ chunk_state,
                           const float* __restrict__ chunk_decay, int heads, int per_head, int chunk_rows, int max_chunks) {
    chain_release();
    chain_wait();
    const size_t state_floats = (size_t)heads * per_head;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (e >= state_floats) return;
    const int h = (int)(e / per_head);
    const int runs = (seq_start[s + 1] - seq_start[s] + chunk_rows - 1) / chunk_rows;
    float cur = state[(size_t)seq_slot[s] * state_stride + e];
    for (int r = 0; r < runs; ++r) {
        const size_t at = (size_t)s * max_chunks + r;
        const float local = r < runs - 1 ? chunk_state[at * state_floats + e] : 0.f;
        chunk_state[at * state_floats + e] = cur;
        if (r < runs - 1) cur = chunk_decay[at * heads + h] * cur + local;
    }
}

// ---------------------------------------------------------------- gate, then norm in groups
// v = y * silu(z); each of `groups` equal parts of the row is divided by its own root mean square
// (eps inside the root) and multiplied by w.  One block per (row, part).
// PER > 0: each thread keeps PER gated values of the part in registers (one read of y and z).
template <typename TO, typename TW, int PER>
__global__ void __launch_bounds__(1024)
gated_group_rmsnorm_kernel(const float* __restrict__ y, int y_stride, const float* __restrict__ z, int z_stride,
                           const TW* __restrict__ w, TO* __restrict__ out, int width, int groups, float eps) {
    chain_release();
    chain_wait();
    __shared__ float scratch[32];
    const int t = blockIdx.x, part = blockIdx.y;
    const int size = width / groups, base = part * size;
    const float* yr = y + (size_t)t * y_stride + base;
    const float* zr = z + (size_t)t * z_stride + base;
    float ss = 0.f;
    if (PER > 0) {
        float v[PER > 0 ? PER : 1];
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            v[i] = e < size ? yr[e] * silu_f(zr[e]) : 0.f;
            ss += v[i] * v[i];
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)size + eps);
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            const int e = i * blockDim.x + threadIdx.x;
            if (e < size) out[(size_t)t * width + base + e] = from_float<TO>(v[i] * scale * to_float(w[base + e]));
        }
    } else {
        for (int e = threadIdx.x; e < size; e += blockDim.x) {
            const float v = yr[e] * silu_f(zr[e]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)size + eps);
        for (int e = threadIdx.x; e < size; e += blockDim.x) {
            const float v = yr[e] * silu_f(zr[e]);
            out[(size_t)t * width + base + e] = from_float<TO>(v * scale * to_float(w[base + e]));
        }
    }
}

}  // namespace mdma

using namespace mdma;

#define MDMA_DISPATCH_2(code_a, TA, code_b, TB, ...) \
    MDMA_DISPATCH_DTYPE(code_a, TA, MDMA_DISPATCH_DTYPE(code_b, TB, __VA_ARGS__))

extern "C" {

int mdma_dyt_norm(const float* x, const void* w, const void* b, const void* alpha, int w_dtype, const int* rows,
                  void* y, int y_dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "dyt_norm: bad sizes");
    if (n_rows == 0) return 0;
    if (width % 4 == 0) {
        MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
            launch_chained(dyt_norm_kernel<TO, TW, 4>, dim3(n_rows, column_parts(width / 4)), dim3(256), 0, stream, x, (const TW*)w,
                           (const TW*)b, (const TW*)alpha, rows, (TO*)y, width));
    } else {
        MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
            launch_chained(dyt_norm_kernel<TO, TW, 1>, dim3(n_rows, column_parts(width)), dim3(256), 0, stream, x, (const TW*)w,
                           (const TW*)b, (const TW*)alpha, rows, (TO*)y, width));
    }
    MDMA_LAUNCH_OK("dyt_norm");
    return 0;
}

int mdma_dyt_shift(const float* x, const void* w, const void* b, const void* alpha, const void* mu, int w_dtype,
                   const int* tok_seq, const int* seq_start, const int* seq_slot, const float* state, long state_stride,
                   void* h, void* hs, int y_dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && state_stride >= width, "dyt_shift: bad sizes");
    if (n_rows == 0) return 0;
    if (width % 4 == 0 && state_stride % 4 == 0 && ((uintptr_t)state & 15) == 0) {
        MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
            launch_chained(dyt_shift_kernel<TO, TW, 4>, dim3(n_rows, column_parts(width / 4)), dim3(256), 0, stream, x, (const TW*)w,
                           (const TW*)b, (const TW*)alpha, (const TW*)mu, tok_seq, seq_start, seq_slot, state, state_stride,
                           (TO*)h, (TO*)hs, width));
    } else {
        MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
            launch_chained(dyt_shift_kernel<TO, TW, 1>, dim3(n_rows, column_parts(width)), dim3(256), 0, stream, x, (const TW*)w,
                           (const TW*)b, (const TW*)alpha, (const TW*)mu, tok_seq, seq_start, seq_slot, state, state_stride,
                           (TO*)h, (TO*)hs, width));
    }
    MDMA_LAUNCH_OK("dyt_shift");
    return 0;
}

int mdma_token_shift(const void* h, int dtype, const void* mu, int mu_dtype, const int* tok_seq, const int* seq_start,
                     const int* seq_slot, const float* state, long state_stride, void* hs, int n_rows, int width,
                     cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && state_stride >= width, "token_shift: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(dtype, T, mu_dtype, TW,
        launch_chained(token_shift_kernel<T, TW>, dim3(n_rows, column_parts(width)), dim3(256), 0, stream, (const T*)h, (const TW*)mu,
                       tok_seq, seq_start, seq_slot, state, state_stride, (T*)hs, width));
    MDMA_LAUNCH_OK("token_shift");
    return 0;
}

int mdma_keep_last_rows(const void* rows, int dtype, const int* seq_start, const int* seq_slot, float* state,
                        long state_stride, int n_seqs, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && width > 0 && state_stride >= width, "keep_last_rows: bad sizes");
    if (n_seqs == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(keep_last_rows_kernel<T>, dim3(n_seqs, column_parts(width)), dim3(256), 0, stream, (const T*)rows, seq_start,
                       seq_slot, state, state_stride, width));
    MDMA_LAUNCH_OK("keep_last_rows");
    return 0;
}

int mdma_gated_add(float* x, const void* g, int g_dtype, const float* y, const float* partial, int splits,
                   long split_stride, int n_rows, int width, const void* keep_rows,
                   int keep_dtype, const int* tok_seq, const int* seq_start, const int* seq_slot, float* state,
                   long state_stride, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "gated_add: bad sizes");
    MDMA_REQUIRE(keep_rows == nullptr || (state != nullptr && state_stride >= width), "gated_add: no place for the kept rows");
    if (n_rows == 0) return 0;
    const bool vec = width % 4 == 0 && split_stride % 4 == 0 && ((uintptr_t)partial & 15) == 0 &&
                     (keep_rows == nullptr || (state_stride % 4 == 0 && ((uintptr_t)state & 15) == 0));
    if (vec) {
        MDMA_DISPATCH_2(g_dtype, TG, keep_dtype, TK,
            launch_chained(gated_add_kernel<TG, TK, 4>, dim3(n_rows, column_parts(width / 4)), dim3(256), 0, stream, x, (const TG*)g, y,
                           partial, partial ? splits : 0, (size_t)split_stride, width, (const TK*)keep_rows, tok_seq, seq_start,
                           seq_slot, state, state_stride));
    } else {
        MDMA_DISPATCH_2(g_dtype, TG, keep_dtype, TK,
            launch_chained(gated_add_kernel<TG, TK, 1>, dim3(n_rows, column_parts(width)), dim3(256), 0, stream, x, (const TG*)g, y,
                           partial, partial ? splits : 0, (size_t)split_stride, width, (const TK*)keep_rows, tok_seq, seq_start,
                           seq_slot, state, state_stride));
    }
    MDMA_LAUNCH_OK("gated_add");
    return 0;
}

int mdma_activation(void* v, int dtype, long n, int act, cudaStream_t stream) {
    MDMA_REQUIRE(n >= 0 && (act == kActSilu || act == kActGeluTanh), "activation: bad arguments");
    if (n == 0) return 0;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    MDMA_DISPATCH_DTYPE(dtype, T, launch_chained(activation_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)v, n, act));
    MDMA_LAUNCH_OK("activation");
    return 0;
}

int mdma_softcap(float* v, long n, float cap, cudaStream_t stream) {
    MDMA_REQUIRE(n >= 0 && cap > 0.f, "softcap: the cap must be positive");
    if (n == 0) return 0;
    const int blocks = (int)((n + 1023) / 1024 < 4096 ? (n + 1023) / 1024 : 4096);
    launch_chained(softcap_kernel, dim3(blocks), dim3(256), 0, stream, v, n, cap);
    MDMA_LAUNCH_OK("softcap");
    return 0;
}

int mdma_pack_pair(const float* a, const float* b, void* out, int dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "pack_pair: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T, launch_chained(pack_pair_kernel<T>, dim3(n_rows, column_parts(width)), dim3(256), 0, stream, a, b, (T*)out, width));
    MDMA_LAUNCH_OK("pack_pair");
    return 0;
}

int mdma_mingru_scan(const float* p, int p_stride, const void* bz, const void* bu, int b_dtype, const int* seq_start,
                     const int* seq_slot, float* state, long state_stride, void* out, int out_dtype, int n_seqs,
                     int width, int chunked, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && width > 0 && p_stride >= 3 * width && state_stride >= width, "mingru_scan: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535, "mingru_scan: too many sequences (%d)", n_seqs);
    if (n_seqs == 0) return 0;
    if (chunked) {
        MDMA_DISPATCH_2(out_dtype, TO, b_dtype, TW,
            launch_chained(mingru_scan_chunked_kernel<TO, TW>, dim3((width + kGruChannels - 1) / kGruChannels, n_seqs),
                           dim3(kGruChunks * kGruChannels), 0, stream, p, p_stride, (const TW*)bz, (const TW*)bu, seq_start,
                           seq_slot, state, state_stride, (TO*)out, width));
        MDMA_LAUNCH_OK("mingru_scan_chunked");
        return 0;
    }
    MDMA_DISPATCH_2(out_dtype, TO, b_dtype, TW,
        launch_chained(mingru_scan_kernel<TO, TW>, dim3((width + 127) / 128, n_seqs), dim3(128), 0, stream, p, p_stride,
                       (const TW*)bz, (const TW*)bu, seq_start, seq_slot, state, state_stride, (TO*)out, width));
    MDMA_LAUNCH_OK("mingru_scan");
    return 0;
}

// `silu` = 0: the convolution's sum with its bias, no activation
int mdma_causal_conv(const float* proj, int proj_stride, int in_col, const void* w, int w_dtype, const void* b,
                     int b_dtype, int taps, int channels, const int* tok_seq, const int* seq_start,
                     const int* seq_slot, float* state, long state_stride, float* out, int n_rows, int n_seqs,
                     int silu, cudaStream_t stream) {
    MDMA_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal_conv: %d taps, the kernel takes 1..%d", taps, kMaxTaps);
    MDMA_REQUIRE(channels > 0 && proj_stride >= in_col + channels && state_stride >= (long)(taps - 1) * channels,
                 "causal_conv: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535, "causal_conv: too many sequences (%d)", n_seqs);
    if (n_rows == 0) return 0;
    if (channels % 4 == 0 && in_col % 4 == 0 && proj_stride % 4 == 0 && state_stride % 4 == 0 &&
        (((uintptr_t)proj | (uintptr_t)state | (uintptr_t)out) & 15) == 0) {
        MDMA_DISPATCH_2(w_dtype, TW, b_dtype, TB,
            launch_chained(causal_conv_silu_kernel<TW, TB, 4>, dim3(n_rows, column_parts(channels / 4)), dim3(256), 0, stream, proj,
                           proj_stride, in_col, (const TW*)w, (const TB*)b, taps, channels, tok_seq, seq_start, seq_slot,
                           (const float*)state, state_stride, out, silu));
    } else {
        MDMA_DISPATCH_2(w_dtype, TW, b_dtype, TB,
            launch_chained(causal_conv_silu_kernel<TW, TB, 1>, dim3(n_rows, column_parts(channels)), dim3(256), 0, stream, proj,
                           proj_stride, in_col, (const TW*)w, (const TB*)b, taps, channels, tok_seq, seq_start, seq_slot,
                           (const float*)state, state_stride, out, silu));
    }
    MDMA_LAUNCH_OK("causal_conv");
    if (taps > 1) {
        launch_chained(conv_keep_kernel, dim3((channels + 255) / 256, n_seqs), dim3(256), 0, stream, proj, proj_stride,
                       in_col, taps, channels, seq_start, seq_slot, state, state_stride);
        MDMA_LAUNCH_OK("conv_keep");
    }
    return 0;
}

int mdma_causal_conv_silu(const float* proj, int proj_stride, int in_col, const void* w, int w_dtype, const void* b,
                          int b_dtype, int taps, int channels, const int* tok_seq, const int* seq_start,
                          const int* seq_slot, float* state, long state_stride, float* out, int n_rows, int n_seqs,
                          cudaStream_t stream) {
    return mdma_causal_conv(proj, proj_stride, in_col, w, w_dtype, b, b_dtype, taps, channels, tok_seq, seq_start, seq_slot,
                            state, state_stride, out, n_rows, n_seqs, 1, stream);
}

// `chunk_rows` > 0: every sequence is walked as runs of that many rows side by side (at most `max_chunks` runs a
// sequence); `scratch` then holds n_seqs * max_chunks * (heads * N * vdim + heads) floats.
int mdma_mamba2_scan(const float* conv, int conv_stride, const float* proj, int proj_stride, int dt_col,
                     const void* dt_bias, const void* A_log, const void* D, int w_dtype, const int* seq_start,
                     const int* seq_slot, float* state, long state_stride, float* y, int n_seqs, int heads, int vdim,
                     int N, int G, int chunk_rows, int max_chunks, float* scratch, long scratch_floats,
                     int wide_state, cudaStream_t stream) {
    MDMA_REQUIRE(heads > 0 && vdim > 0 && N > 0 && G > 0 && heads % G == 0, "mamba2_scan: bad geometry");
    MDMA_REQUIRE(N <= 256, "mamba2_scan: state size %d is beyond the kernel's 256", N);
    MDMA_REQUIRE(state_stride >= (long)(wide_state ? 2 : 1) * heads * N * vdim, "mamba2_scan: the state rows are too short");
    MDMA_REQUIRE(!wide_state || (chunk_rows <= 0 && state_stride % 2 == 0 && ((uintptr_t)state & 7) == 0),
                 "mamba2_scan: a double state goes with the row-by-row walk and rows that start on 8-byte boundaries");
    MDMA_REQUIRE(n_seqs <= 65535 * 1 && heads <= 65535, "mamba2_scan: too many sequences or heads");
    if (n_seqs == 0) return 0;
    const int nper = 8;
    int np = 1;
    while (np * nper < N) np <<= 1;           // lanes per value column: a power of two, at most 32
    const int vpt = vdim >= 32 ? 4 : 1;       // value columns per thread: B and C are fetched once for all of a block's
    const int vb = 128 / np * vpt;
    // two sets of staged rows (B, C, x, raw step sizes), then the step sizes and decays of the set being walked
    const size_t smem = sizeof(float) * 2 * (size_t)(kScanRows * (2 * np * nper + vb + 1)) +
                        (wide_state ? sizeof(double) : sizeof(float)) * 2 * kScanRows;
    dim3 grid(n_seqs, heads, (vdim + vb - 1) / vb);
    MDMA_REQUIRE(grid.z <= 65535, "mamba2_scan: value size %d is too large", vdim);
    float* chunk_state = nullptr;
    float* chunk_decay = nullptr;
    if (chunk_rows > 0) {
        const long state_floats = (long)heads * N * vdim;
        const long slots = (long)n_seqs * max_chunks;
        MDMA_REQUIRE(max_chunks >= 1 && slots <= 65535 * 16l && scratch != nullptr && scratch_floats >= slots * (state_floats + heads),
                     "mamba2_scan: %ld runs need %ld floats of scratch, %ld given", slots, slots * (state_floats + heads), scratch_floats);
        chunk_state = scratch;
        chunk_decay = scratch + slots * state_floats;
        grid.x = (unsigned)slots;
    } else {
        chunk_rows = 0; max_chunks = 1;
    }
#define MDMA_SCAN_LAUNCH_NP(VPT_, NPT_, PASS_, what)                                                                   \
    if (smem > 48 * 1024) {                                                                                            \
        MDMA_DISPATCH_DTYPE(w_dtype, TW,                                                                               \
            cudaFuncSetAttribute(mamba2_scan_kernel<8, VPT_, NPT_, TW, PASS_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    }                                                                                                                  \
    MDMA_DISPATCH_DTYPE(w_dtype, TW,                                                                                   \
        launch_chained(mamba2_scan_kernel<8, VPT_, NPT_, TW, PASS_>, grid, dim3(128), smem, stream, conv, conv_stride,   \
                       proj, proj_stride, dt_col, (const TW*)dt_bias, (const TW*)A_log, (const TW*)D, seq_start, seq_slot, \
                       state, state_stride, y, heads, vdim, N, G, np, chunk_rows, max_chunks, chunk_state, chunk_decay)); \
    MDMA_LAUNCH_OK(what)
#define MDMA_SCAN_LAUNCH(VPT_, PASS_, what)                                                                            \
    if (np == 4) { MDMA_SCAN_LAUNCH_NP(VPT_, 4, PASS_, what); }                                                          \
    else if (np == 8) { MDMA_SCAN_LAUNCH_NP(VPT_, 8, PASS_, what); }                                                     \
    else if (np == 16) { MDMA_SCAN_LAUNCH_NP(VPT_, 16, PASS_, what); }                                                   \
    else { MDMA_SCAN_LAUNCH_NP(VPT_, 0, PASS_, what); }
    if (chunk_rows > 0) {
        if (vpt == 4) { MDMA_SCAN_LAUNCH(4, kScanLocal, "mamba2_scan (runs from zero)"); }
        else { MDMA_SCAN_LAUNCH(1, kScanLocal, "mamba2_scan (runs from zero)"); }
        launch_chained(mamba2_chunk_starts_kernel, dim3((unsigned)(((long)heads * N * vdim + 255) / 256), n_seqs), dim3(256), 0, stream,
                       seq_start, seq_slot, (const float*)state, state_stride, chunk_state, (const float*)chunk_decay, heads,
                       N * vdim, chunk_rows, max_chunks);
        MDMA_LAUNCH_OK("mamba2_chunk_starts");
        if (vpt == 4) { MDMA_SCAN_LAUNCH(4, kScanFrom, "mamba2_scan (runs from their starts)"); }
        else { MDMA_SCAN_LAUNCH(1, kScanFrom, "mamba2_scan (runs from their starts)"); }
        return 0;
    }
    if (wide_state) {
        // the exact engine: state, step sizes, decays and the sums over the state in double
        if (smem > 48 * 1024) {
            MDMA_DISPATCH_DTYPE(w_dtype, TW,
                cudaFuncSetAttribute(mamba2_scan_kernel<8, 4, 0, TW, kScanWhole, double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            MDMA_DISPATCH_DTYPE(w_dtype, TW,
                cudaFuncSetAttribute(mamba2_scan_kernel<8, 1, 0, TW, kScanWhole, double>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        }
        if (vpt == 4) {
            MDMA_DISPATCH_DTYPE(w_dtype, TW,
                launch_chained(mamba2_scan_kernel<8, 4, 0, TW, kScanWhole, double>, grid, dim3(128), smem, stream, conv, conv_stride,
                               proj, proj_stride, dt_col, (const TW*)dt_bias, (const TW*)A_log, (const TW*)D, seq_start, seq_slot,
                               state, state_stride, y, heads, vdim, N, G, np, 0, 1, (float*)nullptr, (float*)nullptr));
        } else {
            MDMA_DISPATCH_DTYPE(w_dtype, TW,
                launch_chained(mamba2_scan_kernel<8, 1, 0, TW, kScanWhole, double>, grid, dim3(128), smem, stream, conv, conv_stride,
                               proj, proj_stride, dt_col, (const TW*)dt_bias, (const TW*)A_log, (const TW*)D, seq_start, seq_slot,
                               state, state_stride, y, heads, vdim, N, G, np, 0, 1, (float*)nullptr, (float*)nullptr));
        }
        MDMA_LAUNCH_OK("mamba2_scan (double state)");
        return 0;
    }
    if (vpt == 4) { MDMA_SCAN_LAUNCH(4, kScanWhole, "mamba2_scan"); }
    else { MDMA_SCAN_LAUNCH(1, kScanWhole, "mamba2_scan"); }
#undef MDMA_SCAN_LAUNCH
#undef MDMA_SCAN_LAUNCH_NP
    return 0;
}

int mdma_gated_group_rmsnorm(const float* y, int y_stride, const float* z, int z_stride, const void* w, int w_dtype,
                             void* out, int out_dtype, int n_rows, int width, int groups, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(width > 0 && groups > 0 && width % groups == 0, "gated_group_rmsnorm: %d columns in %d parts", width, groups);
    MDMA_REQUIRE(groups <= 65535, "gated_group_rmsnorm: too many parts");
    if (n_rows == 0) return 0;
    const int size = width / groups;
    if (size <= 1024) {
        MDMA_DISPATCH_2(out_dtype, TO, w_dtype, TW,
            launch_chained(gated_group_rmsnorm_kernel<TO, TW, 4>, dim3(n_rows, groups), dim3(256), 0, stream, y, y_stride, z,
                           z_stride, (const TW*)w, (TO*)out, width, groups, eps));
    } else if (size <= 8192) {
        MDMA_DISPATCH_2(out_dtype, TO, w_dtype, TW,
            launch_chained(gated_group_rmsnorm_kernel<TO, TW, 8>, dim3(n_rows, groups), dim3(1024), 0, stream, y, y_stride, z,
                           z_stride, (const TW*)w, (TO*)out, width, groups, eps));
    } else {
        MDMA_DISPATCH_2(out_dtype, TO, w_dtype, TW,
            launch_chained(gated_group_rmsnorm_kernel<TO, TW, 0>, dim3(n_rows, groups), dim3(1024), 0, stream, y, y_stride, z,
                           z_stride, (const TW*)w, (TO*)out, width, groups, eps));
    }
    MDMA_LAUNCH_OK("gated_group_rmsnorm");
    return 0;
}

}  // extern "C"
