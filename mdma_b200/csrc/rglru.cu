// The real-gated linear recurrent unit, and the small row kernels of the layers around it:
// a layer norm with a weight and no bias, the re-entry of a looped stack by addition, a
// per-row scale and an element-wise sigmoid gate.
//
// The recurrence, per channel c of a sequence, row by row:
//     r = sigmoid(rp + rb[c]),  i = sigmoid(ip + ib[c])          (rp, ip: the gates' block-diagonal products)
//     log a = -decay * r * softplus(lam[c]),  a = exp(log a)
//     S = a S + sqrt(1 - a^2) (i u)
//     out = S * gelu_tanh(y)
// u is the convolved input branch, y the other branch before its activation.  Everything is float
// in both engines; the state S is float, one number per channel and sequence.  1 - a^2 is taken as
// -expm1(2 log a): the difference of two numbers near one would lose the digits that matter when a
// gate is almost closed.
//
// The step's tokens are a flat batch: sequence s owns rows [seq_start[s], seq_start[s+1]) and keeps
// its state in row seq_slot[s] of the state tensor.
#include "common.cuh"

namespace mdma {

__device__ __forceinline__ float lru_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float lru_softplus(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

struct LruRow {
    const float* gates_r;      // [T, width] the recurrence gate's product
    const float* gates_i;      // [T, width] the input gate's product
    const float* u;            // [T, width] the convolved branch
    const float* y;            // rows `y_stride` apart: the other branch before its activation
    int y_stride;
};

// a_t and b_t of S_t = a_t S_(t-1) + b_t for one row and channel
__device__ __forceinline__ void lru_coefficients(const LruRow& in, size_t t, int c, int width, float rb, float ib,
                                                 float neg_decay_softplus, float& a, float& b) {
    const size_t e = t * width + c;
    const float r = lru_sigmoid(in.gates_r[e] + rb);
    const float i = lru_sigmoid(in.gates_i[e] + ib);
    const float log_a = neg_decay_softplus * r;
    a = expf(log_a);
    b = sqrtf(-expm1f(2.0f * log_a)) * (i * in.u[e]);
}

template <typename TO, typename TW>
__global__ void __launch_bounds__(128)
rglru_scan_kernel(const LruRow in, const TW* __restrict__ rb, const TW* __restrict__ ib, const TW* __restrict__ lam,
                  float decay, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                  float* __restrict__ state, long state_stride, TO* __restrict__ out, int width) {
    chain_release();
    chain_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int s = blockIdx.y;
    if (c >= width) return;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    const float rbc = to_float(rb[c]), ibc = to_float(ib[c]);
    const float nds = -decay * lru_softplus(to_float(lam[c]));
    float* kept = state + (size_t)seq_slot[s] * state_stride + c;
    float S = *kept;
    for (int t = t0; t < t1; ++t) {
        float a, b;
        lru_coefficients(in, (size_t)t, c, width, rbc, ibc, nds, a, b);
        S = fmaf(a, S, b);
        out[(size_t)t * width + c] = from_float<TO>(S * gate_activation(in.y[(size_t)t * in.y_stride + c], kActGeluTanh));
    }
    *kept = S;
}

// Steps that bring many rows per sequence: the recurrence is linear in S, so a sequence's rows are cut into
// kLruRuns runs that are walked side by side.  A thread walks one run of one channel from zero and keeps the
// run's product of a and its last value; the runs' starting values follow from those in order; every run is
// walked again from its starting value and writes its outputs.  Equal to the row-by-row walk up to rounding:
// the serving engine uses it for long prompts, the 32-bit engine never.
constexpr int kLruRuns = 128, kLruChannels = 8;

template <typename TO, typename TW>
__global__ void __launch_bounds__(kLruRuns * kLruChannels)
rglru_scan_runs_kernel(const LruRow in, const TW* __restrict__ rb, const TW* __restrict__ ib, const TW* __restrict__ lam,
                       float decay, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                       float* __restrict__ state, long state_stride, TO* __restrict__ out, int width) {
    chain_release();
    chain_wait();
    __shared__ float sA[kLruRuns][kLruChannels], sB[kLruRuns][kLruChannels];
    const int lane_c = threadIdx.x % kLruChannels, k = threadIdx.x / kLruChannels;
    const int c = blockIdx.x * kLruChannels + lane_c;
    const int s = blockIdx.y;
    const bool live = c < width;
    const int t0 = seq_start[s], t1 = seq_start[s + 1];
    const int run = (t1 - t0 + kLruRuns - 1) / kLruRuns;
    const int lo = min(t1, t0 + k * run), hi = min(t1, lo + run);
    const float rbc = live ? to_float(rb[c]) : 0.f, ibc = live ? to_float(ib[c]) : 0.f;
    const float nds = live ? -decay * lru_softplus(to_float(lam[c])) : 0.f;
    float A = 1.f, B = 0.f;
    if (live) {
        for (int t = lo; t < hi; ++t) {
            float a, b;
            lru_coefficients(in, (size_t)t, c, width, rbc, ibc, nds, a, b);
            A *= a;
            B = fmaf(a, B, b);
        }
    }
    sA[k][lane_c] = A;
    sB[k][lane_c] = B;
    __syncthreads();
    if (k == 0 && live) {
        float* kept = state + (size_t)seq_slot[s] * state_stride + c;
        float S = *kept;
        for (int j = 0; j < kLruRuns; ++j) {
            const float next = fmaf(sA[j][lane_c], S, sB[j][lane_c]);
            sB[j][lane_c] = S;                       // the run's starting value
            S = next;
        }
        *kept = S;
    }
    __syncthreads();
    if (live) {
        float S = sB[k][lane_c];
        for (int t = lo; t < hi; ++t) {
            float a, b;
            lru_coefficients(in, (size_t)t, c, width, rbc, ibc, nds, a, b);
            S = fmaf(a, S, b);
            out[(size_t)t * width + c] = from_float<TO>(S * gate_activation(in.y[(size_t)t * in.y_stride + c], kActGeluTanh));
        }
    }
}

// ---------------------------------------------------------------- layer norm, weight only
// y[r,:] = (x[src,:] - mean) / sqrt(var + eps) * w, var the mean of the squared deviations; src = rows[r] or r.
// One block per row.  The row is read from memory once and kept in shared memory (STAGED) for the two further passes;
// rows too long for that are read three times.  Sums in float, fixed order.
template <typename TO, typename TW, bool STAGED>
__global__ void __launch_bounds__(1024)
layernorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, const int* __restrict__ rows,
                 TO* __restrict__ y, int width, float eps) {
    chain_release();
    chain_wait();
    extern __shared__ __align__(16) float staged_row[];
    __shared__ float scratch[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * width;
    float sum = 0.f;
    if (STAGED && width % 4 == 0 && ((uintptr_t)xr & 15) == 0) {
        for (int e = threadIdx.x * 4; e < width; e += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(xr + e);
            *reinterpret_cast<float4*>(staged_row + e) = v;
            sum += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int e = threadIdx.x; e < width; e += blockDim.x) {
            const float v = xr[e];
            if (STAGED) staged_row[e] = v;
            sum += v;
        }
    }
    const float* row = STAGED ? staged_row : xr;
    const float mean = block_sum(sum, scratch) / (float)width;      // (its barriers also publish the staged row)
    float sq = 0.f;
    for (int e = threadIdx.x; e < width; e += blockDim.x) {
        const float d = row[e] - mean;
        sq = fmaf(d, d, sq);
    }
    const float var = block_sum(sq, scratch) / (float)width;
    const float inv = 1.0f / sqrtf(var + eps);
    TO* yr = y + (size_t)r * width;
    for (int e = threadIdx.x; e < width; e += blockDim.x)
        yr[e] = from_float<TO>((row[e] - mean) * inv * to_float(w[e]));
}

// ---------------------------------------------------------------- re-entry of a looped stack by addition
// x[t,:] = (x[t,:] + x0[t,:]) + step[:]   (x0 null: the first pass, only the step vector is added)
template <typename TW>
__global__ void __launch_bounds__(256)
loop_add_kernel(float* __restrict__ x, const float* __restrict__ x0, const TW* __restrict__ step, long n, int width) {
    chain_release();
    chain_wait();
    for (long e = (long)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
        float v = x[e];
        if (x0) v += x0[e];
        x[e] = v + to_float(step[e % width]);
    }
}

// ---------------------------------------------------------------- v[t,:] *= s[t]
template <typename T>
__global__ void __launch_bounds__(256)
scale_rows_kernel(T* __restrict__ v, const float* __restrict__ s, int width) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    const float f = s[t];
    T* row = v + (size_t)t * width;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x)
        row[e] = from_float<T>(to_float(row[e]) * f);
}

// ---------------------------------------------------------------- v[t,:] *= sigmoid(g[t,:])
template <typename T>
__global__ void __launch_bounds__(256)
sigmoid_gate_kernel(T* __restrict__ v, const T* __restrict__ g, int g_stride, int width) {
    chain_release();
    chain_wait();
    const int t = blockIdx.x;
    T* row = v + (size_t)t * width;
    const T* gate = g + (size_t)t * g_stride;
    for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < width; e += gridDim.y * blockDim.x)
        row[e] = from_float<T>(to_float(row[e]) / (1.0f + expf(-to_float(gate[e]))));
}

}  // namespace mdma

using namespace mdma;

extern "C" {

// gates_r, gates_i, u: [T, width] floats; y: float rows y_stride apart; rb, ib, lam: [width] of one dtype;
// state rows are state_stride floats apart; runs != 0: the side-by-side walk.
int mdma_rglru_scan(const float* gates_r, const float* gates_i, const float* u, const float* y, int y_stride,
                    const void* rb, const void* ib, const void* lam, int w_dtype, float decay, const int* seq_start,
                    const int* seq_slot, float* state, long state_stride, void* out, int out_dtype, int n_seqs,
                    int width, int runs, cudaStream_t stream) {
    MDMA_REQUIRE(n_seqs >= 0 && width > 0 && n_seqs <= 65535 && decay > 0.f, "rglru_scan: bad sizes");
    if (n_seqs == 0) return 0;
    const LruRow in{gates_r, gates_i, u, y, y_stride};
    MDMA_DISPATCH_DTYPE(out_dtype, TO,
        MDMA_DISPATCH_DTYPE(w_dtype, TW,
            if (runs)
                launch_chained(rglru_scan_runs_kernel<TO, TW>, dim3((width + kLruChannels - 1) / kLruChannels, n_seqs),
                               dim3(kLruRuns * kLruChannels), 0, stream, in, (const TW*)rb, (const TW*)ib, (const TW*)lam,
                               decay, seq_start, seq_slot, state, state_stride, (TO*)out, width);
            else
                launch_chained(rglru_scan_kernel<TO, TW>, dim3((width + 127) / 128, n_seqs), dim3(128), 0, stream, in,
                               (const TW*)rb, (const TW*)ib, (const TW*)lam, decay, seq_start, seq_slot, state,
                               state_stride, (TO*)out, width)));
    MDMA_LAUNCH_OK("rglru_scan");
    return 0;
}

int mdma_layernorm(const float* x, const void* w, int w_dtype, const int* rows, void* y, int y_dtype, int n_rows,
                   int width, float eps, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "layernorm: bad sizes");
    if (n_rows == 0) return 0;
    // 256 threads up to 2,048 columns, 512 up to 8,192 (1,024 were slower at 4,096: 29.0 against 17.8 us for 2,048
    // rows), 1,024 beyond; the row staged while it fits 48 KB of shared memory
    const int threads = width <= 2048 ? 256 : width <= 8192 ? 512 : 1024;
    const size_t staged = (size_t)width * sizeof(float);
    MDMA_DISPATCH_DTYPE(y_dtype, TO,
        MDMA_DISPATCH_DTYPE(w_dtype, TW,
            if (staged <= 48 * 1024)
                launch_chained(layernorm_kernel<TO, TW, true>, dim3(n_rows), dim3(threads), staged, stream, x, (const TW*)w, rows,
                               (TO*)y, width, eps);
            else
                launch_chained(layernorm_kernel<TO, TW, false>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w, rows,
                               (TO*)y, width, eps)));
    MDMA_LAUNCH_OK("layernorm");
    return 0;
}

int mdma_loop_add(float* x, const float* x0, const void* step, int step_dtype, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "loop_add: bad sizes");
    if (n_rows == 0) return 0;
    const long n = (long)n_rows * width;
    const unsigned blocks = (unsigned)((n + 255) / 256 > 4096 ? 4096 : (n + 255) / 256);
    MDMA_DISPATCH_DTYPE(step_dtype, TW,
        launch_chained(loop_add_kernel<TW>, dim3(blocks), dim3(256), 0, stream, x, x0, (const TW*)step, n, width));
    MDMA_LAUNCH_OK("loop_add");
    return 0;
}

int mdma_scale_rows(void* v, int dtype, const float* s, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0, "scale_rows: bad sizes");
    if (n_rows == 0) return 0;
    const int parts = (width + 255) / 256;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(scale_rows_kernel<T>, dim3(n_rows, parts > 64 ? 64 : parts), dim3(256), 0, stream, (T*)v, s, width));
    MDMA_LAUNCH_OK("scale_rows");
    return 0;
}

int mdma_sigmoid_gate(void* v, const void* g, int dtype, int g_stride, int n_rows, int width, cudaStream_t stream) {
    MDMA_REQUIRE(n_rows >= 0 && width > 0 && g_stride >= width, "sigmoid_gate: bad sizes");
    if (n_rows == 0) return 0;
    const int parts = (width + 255) / 256;
    MDMA_DISPATCH_DTYPE(dtype, T,
        launch_chained(sigmoid_gate_kernel<T>, dim3(n_rows, parts > 64 ? 64 : parts), dim3(256), 0, stream, (T*)v, (const T*)g,
                       g_stride, width));
    MDMA_LAUNCH_OK("sigmoid_gate");
    return 0;
}

}  // extern "C"
