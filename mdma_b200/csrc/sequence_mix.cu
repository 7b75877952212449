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

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

// ---------------------------------------------------------------- dynamic tanh
// y[r,:] = tanh(alpha * x[src,:]) * w + b, src = rows[r] or r.  No sum over the row.
template <typename TO, typename TW>
__global__ void __launch_bounds__(256)
dyt_norm_kernel(const float* __restrict__ x, const TW* __restrict__ w, const TW* __restrict__ b,
                const TW* __restrict__ alpha, const int* __restrict__ rows, TO* __restrict__ y, int width) {
    chain_release();
    chain_wait();
    const int r = blockIdx.x;
    const float a = to_float(alpha[0]);
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    TO* yr = y + (size_t)r * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        yr[e] = from_float<TO>(tanhf(a * xr[e]) * to_float(w[e]) + to_float(b[e]));
}

// The same with the token shift behind it: h = dyt(x[t]) and hs = h + (h' - h) * mu, h' the h of the
// row before in the same sequence (recomputed from x, which costs nothing for a norm without sums) or,
// for a sequence's first row of the step, the kept one.  Both h and h' are rounded to the activation
// type first, so that the kept value and the recomputed one are the same number.
template <typename TO, typename TW>
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
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float we = to_float(w[e]), be = to_float(b[e]);
        const float cur = to_float(from_float<TO>(tanhf(a * xr[e]) * we + be));
        const float before = first ? prev[e] : to_float(from_float<TO>(tanhf(a * prev[e]) * we + be));
        h[(size_t)t * width + e] = from_float<TO>(cur);
        hs[(size_t)t * width + e] = from_float<TO>(cur + (before - cur) * to_float(mu[e]));
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
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
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
    for (int e = threadIdx.x; e < width; e += blockDim.x) kept[e] = to_float(last[e]);
}

// ---------------------------------------------------------------- gated residual add
// x[t,:] += sigmoid(g[t,:]) * y[t,:].  With `keep` the rows of `keep_rows` that end a sequence go to
// the state as well (the token shift's kept row), which saves a launch.
template <typename TG, typename TK>
__global__ void __launch_bounds__(256)
gated_add_kernel(float* __restrict__ x, const TG* __restrict__ g, const float* __restrict__ y, int width,
                 const TK* __restrict__ keep_rows, const int* __restrict__ tok_seq, const int* __restrict__ seq_start,
                 const int* __restrict__ seq_slot, float* __restrict__ state, long state_stride) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const size_t o = (size_t)t * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        x[o + e] = x[o + e] + sigmoid_f(to_float(g[o + e])) * y[o + e];
    if (keep_rows != nullptr) {
        const int s = tok_seq[t];
        if (t == seq_start[s + 1] - 1) {
            float* kept = state + (size_t)seq_slot[s] * state_stride;
            for (int e = threadIdx.x; e < width; e += blockDim.x) kept[e] = to_float(keep_rows[o + e]);
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
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
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

// ---------------------------------------------------------------- short causal convolution
// out[t,c] = silu(sum_j w[c,j] * in(t - (taps-1) + j, c) + b[c]); in(.) is column in_col + c of the
// projection rows of this step, or, before the step's first row of the sequence, the kept inputs
// (`state`: [taps-1, channels] floats per slot, oldest first; zeros before the sequence's start).
template <typename TW, typename TB>
__global__ void __launch_bounds__(256)
causal_conv_silu_kernel(const float* __restrict__ proj, int proj_stride, int in_col, const TW* __restrict__ w,
                        const TB* __restrict__ b, int taps, int channels, const int* __restrict__ tok_seq,
                        const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                        const float* __restrict__ state, long state_stride, float* __restrict__ out) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const int s = tok_seq[t];
    const int t0 = seq_start[s];
    const float* kept = state + (size_t)seq_slot[s] * state_stride;
    for (int c = threadIdx.x; c < channels; c += blockDim.x) {
        float acc = to_float(b[c]);
        for (int j = 0; j < taps; ++j) {
            const int src = t - (taps - 1) + j;            // a row of this step, or before it
            const float v = src >= t0 ? proj[(size_t)src * proj_stride + in_col + c]
                                      : kept[(size_t)(taps - 1 + (src - t0)) * channels + c];
            acc = fmaf(to_float(w[(size_t)c * taps + j]), v, acc);
        }
        out[(size_t)t * channels + c] = silu_f(acc);
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
// memory sixteen at a time.  The state of a (sequence, head, column) is read and written by the same threads.
constexpr int kScanRows = 16;

template <int NPER, typename TW>
__global__ void __launch_bounds__(128)
mamba2_scan_kernel(const float* __restrict__ conv, int conv_stride, const float* __restrict__ proj, int proj_stride,
                   int dt_col, const TW* __restrict__ dt_bias, const TW* __restrict__ A_log, const TW* __restrict__ D,
                   const int* __restrict__ seq_start, const int* __restrict__ seq_slot, float* __restrict__ state,
                   long state_stride, float* __restrict__ y, int heads, int vdim, int N, int G, int NP) {
    chain_release();
    chain_wait();
    extern __shared__ float sm[];
    const int VB = blockDim.x / NP;
    const int Npad = NP * NPER;
    float* sB = sm;
    float* sC = sB + kScanRows * Npad;
    float* sx = sC + kScanRows * Npad;
    float* sdt = sx + kScanRows * VB;
    float* sa = sdt + kScanRows;
    const int s = blockIdx.x, h = blockIdx.y, v0 = blockIdx.z * VB;
    const int g = h / (heads / G);
    const int np = threadIdx.x % NP, vl = threadIdx.x / NP;
    const int v = v0 + vl;
    const bool vok = v < vdim;
    const int inner = heads * vdim;
    float* Sg = state + (size_t)seq_slot[s] * state_stride + (size_t)h * N * vdim;
    float S[NPER];
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = np * NPER + i;
        S[i] = (vok && n < N) ? Sg[(size_t)n * vdim + v] : 0.f;
    }
    const float rate = expf(to_float(A_log[h])), Dh = to_float(D[h]), bias = to_float(dt_bias[h]);
    const int t_begin = seq_start[s], t_end = seq_start[s + 1];
    for (int t0 = t_begin; t0 < t_end; t0 += kScanRows) {
        const int nt = min(kScanRows, t_end - t0);
        __syncthreads();
        for (int i = threadIdx.x; i < nt * Npad; i += blockDim.x) {
            const int tt = i / Npad, n = i % Npad;
            const float* row = conv + (size_t)(t0 + tt) * conv_stride + inner + g * N;
            sB[i] = n < N ? row[n] : 0.f;
            sC[i] = n < N ? row[G * N + n] : 0.f;
        }
        for (int i = threadIdx.x; i < nt * VB; i += blockDim.x) {
            const int tt = i / VB, vv = i % VB;
            sx[i] = (v0 + vv < vdim) ? conv[(size_t)(t0 + tt) * conv_stride + h * vdim + v0 + vv] : 0.f;
        }
        for (int i = threadIdx.x; i < nt; i += blockDim.x) {
            const float d = softplus_f(proj[(size_t)(t0 + i) * proj_stride + dt_col + h] + bias);
            sdt[i] = d;
            sa[i] = expf(-rate * d);
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float a = sa[tt], xv = sx[tt * VB + vl], dtx = sdt[tt] * xv;
            const float* Bt = sB + tt * Npad + np * NPER;
            const float* Ct = sC + tt * Npad + np * NPER;
            float acc = 0.f;
#pragma unroll
            for (int i = 0; i < NPER; ++i) {
                S[i] = fmaf(a, S[i], dtx * Bt[i]);
                acc = fmaf(S[i], Ct[i], acc);
            }
            for (int o = NP >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            if (np == 0 && vok) y[(size_t)(t0 + tt) * inner + h * vdim + v] = acc + Dh * xv;
        }
    }
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
        const int n = np * NPER + i;
        if (vok && n < N) Sg[(size_t)n * vdim + v] = S[i];
    }
}

// ---------------------------------------------------------------- gate, then norm in groups
// v = y * silu(z); each of `groups` equal parts of the row is divided by its own root mean square
// (eps inside the root) and multiplied by w.  One block per (row, part).
template <typename TO, typename TW>
__global__ void __launch_bounds__(256)
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

}  // namespace mdma

using namespace mdma;

#define MDMA_DISPATCH_2(code_a, TA, code_b, TB, ...) \
    MDMA_DISPATCH_DTYPE(code_a, TA, MDMA_DISPATCH_DTYPE(code_b, TB, __VA_ARGS__))

extern "C" {

int mdma_dyt_norm(const float* x, const void* w, const void* b, const void* alpha, int w_dtype, const int* rows,
                  void* y, int y_dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "dyt_norm: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
        launch_chained(dyt_norm_kernel<TO, TW>, dim3(n_rows), dim3(256), 0, stream, x, (const TW*)w, (const TW*)b,
                       (const TW*)alpha, rows, (TO*)y, width));
    MDMA_LAUNCH_OK("dyt_norm");
    return 0;
}

int mdma_dyt_shift(const float* x, const void* w, const void* b, const void* alpha, const void* mu, int w_dtype,
                   const int* tok_seq, const int* seq_start, const int* seq_slot, const float* state, long state_stride,
                   void* h, void* hs, int y_dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && state_stride >= width, "dyt_shift: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(y_dtype, TO, w_dtype, TW,
        launch_chained(dyt_shift_kernel<TO, TW>, dim3(n_rows), dim3(256), 0, stream, x, (const TW*)w, (const TW*)b,
                       (const TW*)alpha, (const TW*)mu, tok_seq, seq_start, seq_slot, state, state_stride,
                       (TO*)h, (TO*)hs, width));
    MDMA_LAUNCH_OK("dyt_shift");
    return 0;
}

int mdma_token_shift(const void* h, int dtype, const void* mu, int mu_dtype, const int* tok_seq, const int* seq_start,
                     const int* seq_slot, const float* state, long state_stride, void* hs, int n_rows, int width,
                     cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && state_stride >= width, "token_shift: bad sizes");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(dtype, T, mu_dtype, TW,
        launch_chained(token_shift_kernel<T, TW>, dim3(n_rows), dim3(256), 0, stream, (const T*)h, (const TW*)mu,
                       tok_seq, seq_start, seq_slot, state, state_stride, (T*)hs, width));
    MDMA_LAUNCH_OK("token_shift");
    return 0;
}

int mdma_keep_last_rows(const void* rows, int dtype, const int* seq_start, const int* seq_slot, float* state,
                        long state_stride, int n_seqs, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && width > 0 && state_stride >= width, "keep_last_rows: bad sizes");
    if (n_seqs == 0) return 0;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(keep_last_rows_kernel<T>, dim3(n_seqs), dim3(256), 0, stream, (const T*)rows, seq_start,
                       seq_slot, state, state_stride, width));
    MDMA_LAUNCH_OK("keep_last_rows");
    return 0;
}

int mdma_gated_add(float* x, const void* g, int g_dtype, const float* y, int n_rows, int width, const void* keep_rows,
                   int keep_dtype, const int* tok_seq, const int* seq_start, const int* seq_slot, float* state,
                   long state_stride, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "gated_add: bad sizes");
    MDMA_REQUIRE(keep_rows == nullptr || (state != nullptr && state_stride >= width), "gated_add: no place for the kept rows");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(g_dtype, TG, keep_dtype, TK,
        launch_chained(gated_add_kernel<TG, TK>, dim3(n_rows), dim3(256), 0, stream, x, (const TG*)g, y, width,
                       (const TK*)keep_rows, tok_seq, seq_start, seq_slot, state, state_stride));
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
    MDMA_DISPATCH_DTYPE(dtype, T, launch_chained(pack_pair_kernel<T>, dim3(n_rows), dim3(256), 0, stream, a, b, (T*)out, width));
    MDMA_LAUNCH_OK("pack_pair");
    return 0;
}

int mdma_mingru_scan(const float* p, int p_stride, const void* bz, const void* bu, int b_dtype, const int* seq_start,
                     const int* seq_slot, float* state, long state_stride, void* out, int out_dtype, int n_seqs,
                     int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && width > 0 && p_stride >= 3 * width && state_stride >= width, "mingru_scan: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535, "mingru_scan: too many sequences (%d)", n_seqs);
    if (n_seqs == 0) return 0;
    MDMA_DISPATCH_2(out_dtype, TO, b_dtype, TW,
        launch_chained(mingru_scan_kernel<TO, TW>, dim3((width + 127) / 128, n_seqs), dim3(128), 0, stream, p, p_stride,
                       (const TW*)bz, (const TW*)bu, seq_start, seq_slot, state, state_stride, (TO*)out, width));
    MDMA_LAUNCH_OK("mingru_scan");
    return 0;
}

int mdma_causal_conv_silu(const float* proj, int proj_stride, int in_col, const void* w, int w_dtype, const void* b,
                          int b_dtype, int taps, int channels, const int* tok_seq, const int* seq_start,
                          const int* seq_slot, float* state, long state_stride, float* out, int n_rows, int n_seqs,
                          cudaStream_t stream) {
    MDMA_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal_conv: %d taps, the kernel takes 1..%d", taps, kMaxTaps);
    MDMA_REQUIRE(channels > 0 && proj_stride >= in_col + channels && state_stride >= (long)(taps - 1) * channels,
                 "causal_conv: bad sizes");
    MDMA_REQUIRE(n_seqs <= 65535, "causal_conv: too many sequences (%d)", n_seqs);
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(w_dtype, TW, b_dtype, TB,
        launch_chained(causal_conv_silu_kernel<TW, TB>, dim3(n_rows), dim3(256), 0, stream, proj, proj_stride, in_col,
                       (const TW*)w, (const TB*)b, taps, channels, tok_seq, seq_start, seq_slot, (const float*)state,
                       state_stride, out));
    MDMA_LAUNCH_OK("causal_conv_silu");
    if (taps > 1) {
        launch_chained(conv_keep_kernel, dim3((channels + 255) / 256, n_seqs), dim3(256), 0, stream, proj, proj_stride,
                       in_col, taps, channels, seq_start, seq_slot, state, state_stride);
        MDMA_LAUNCH_OK("conv_keep");
    }
    return 0;
}

int mdma_mamba2_scan(const float* conv, int conv_stride, const float* proj, int proj_stride, int dt_col,
                     const void* dt_bias, const void* A_log, const void* D, int w_dtype, const int* seq_start,
                     const int* seq_slot, float* state, long state_stride, float* y, int n_seqs, int heads, int vdim,
                     int N, int G, cudaStream_t stream) {
    MDMA_REQUIRE(heads > 0 && vdim > 0 && N > 0 && G > 0 && heads % G == 0, "mamba2_scan: bad geometry");
    MDMA_REQUIRE(N <= 256, "mamba2_scan: state size %d is beyond the kernel's 256", N);
    MDMA_REQUIRE(state_stride >= (long)heads * N * vdim, "mamba2_scan: the state rows are too short");
    MDMA_REQUIRE(n_seqs <= 65535 * 1 && heads <= 65535, "mamba2_scan: too many sequences or heads");
    if (n_seqs == 0) return 0;
    const int nper = 8;
    int np = 1;
    while (np * nper < N) np <<= 1;           // lanes per value column: a power of two, at most 32
    const int vb = 128 / np;
    const size_t smem = sizeof(float) * (size_t)(2 * kScanRows * np * nper + kScanRows * vb + 2 * kScanRows);
    dim3 grid(n_seqs, heads, (vdim + vb - 1) / vb);
    MDMA_REQUIRE(grid.z <= 65535, "mamba2_scan: value size %d is too large", vdim);
    MDMA_DISPATCH_DTYPE(w_dtype, TW,
        launch_chained(mamba2_scan_kernel<8, TW>, grid, dim3(128), smem, stream, conv, conv_stride, proj, proj_stride,
                       dt_col, (const TW*)dt_bias, (const TW*)A_log, (const TW*)D, seq_start, seq_slot, state,
                       state_stride, y, heads, vdim, N, G, np));
    MDMA_LAUNCH_OK("mamba2_scan");
    return 0;
}

int mdma_gated_group_rmsnorm(const float* y, int y_stride, const float* z, int z_stride, const void* w, int w_dtype,
                             void* out, int out_dtype, int n_rows, int width, int groups, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(width > 0 && groups > 0 && width % groups == 0, "gated_group_rmsnorm: %d columns in %d parts", width, groups);
    MDMA_REQUIRE(groups <= 65535, "gated_group_rmsnorm: too many parts");
    if (n_rows == 0) return 0;
    MDMA_DISPATCH_2(out_dtype, TO, w_dtype, TW,
        launch_chained(gated_group_rmsnorm_kernel<TO, TW>, dim3(n_rows, groups), dim3(256), 0, stream, y, y_stride, z,
                       z_stride, (const TW*)w, (TO*)out, width, groups, eps));
    MDMA_LAUNCH_OK("gated_group_rmsnorm");
    return 0;
}

}  // extern "C"
