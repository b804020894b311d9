// A mixture of small gated feed-forward units: the router, and the experts' products for the experts that each row
// chose.  The experts' matrices are stacked and stored (out, in), so that an output element is one dot product over
// contiguous weights; a kernel finds an expert's matrix from the row's choice on the device, nothing is sorted or
// gathered.  Sums are 32-bit; T is the storage type of activations and weights.
#include "common.cuh"

namespace {

constexpr int MOE_THREADS = 128;

// sum_i w[i] * xs[i] over a warp: 16-byte loads of the weights when `vec` (d a multiple of a vector, w aligned).
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const float* __restrict__ xs, int d, int lane, bool vec) {
    constexpr int N = Vec16<T>::N;
    float acc = 0.f;
    if (vec) {
        float v[N];
        for (int i = lane * N; i < d; i += 32 * N) {
            Vec16<T>::load(w + i, v);
#pragma unroll
            for (int e = 0; e < N; ++e) acc = fmaf(v[e], xs[i + e], acc);
        }
    } else {
        for (int i = lane; i < d; i += 32) acc = fmaf(to_f32(w[i]), xs[i], acc);
    }
    return warp_sum(acc);
}

// ------------------------------------------------------------------------------------------------------------
// The router, a CTA a row:  s = sigmoid(W x) over E experts (W float32 (E, d));  pick = s + correction;  with
// groups > 0 the experts form that many groups of E / groups neighbours, a group's strength is the sum of its two
// largest picks, and only the experts of the `keep` strongest groups stay in the race;  the `top` largest picks
// win (the lower index on a tie);  weights: their s over the sum of those (+ weight_eps).  Also sigmoid(w_sg . x)
// if w_sg is given.
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_route_kernel(const T* __restrict__ x, int ldx, const float* __restrict__ wr, const float* __restrict__ corr,
                 const float* __restrict__ w_sg, int d, int E, int groups, int keep, int top, float weight_eps,
                 int* __restrict__ chosen, float* __restrict__ weights, float* __restrict__ shared_gate) {
    extern __shared__ float smem[];
    float* xs = smem;                  // [d]
    float* sc = xs + d;                // [E]  sigmoid scores
    float* pick = sc + E;              // [E]  choosing scores; -inf once out of the race
    float* strength = pick + E;        // [groups]
    pdl_launch_dependents();
    const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    for (int i = tid; i < d; i += blockDim.x) xs[i] = to_f32(x[(size_t)r * ldx + i]);
    __syncthreads();
    const bool vec = d % 4 == 0;
    for (int e = warp; e < E + (w_sg != nullptr ? 1 : 0); e += nw) {
        const float z = warp_dot<float>(e < E ? wr + (size_t)e * d : w_sg, xs, d, lane, vec);
        if (lane == 0) {
            const float s = 1.f / (1.f + expf(-z));
            if (e < E) { sc[e] = s; pick[e] = s + (corr != nullptr ? corr[e] : 0.f); }
            else shared_gate[r] = s;
        }
    }
    __syncthreads();
    if (tid != 0) return;
    if (groups > 0) {
        const int per = E / groups;
        for (int g = 0; g < groups; ++g) {
            float a = -INFINITY, b = -INFINITY;            // the two largest picks of the group
            for (int i = 0; i < per; ++i) {
                const float v = pick[g * per + i];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            strength[g] = per > 1 ? a + b : a;
        }
        // the `keep` strongest groups stay; a kept group's strength is set to +inf as its mark
        for (int k = 0; k < keep; ++k) {
            int best = -1;
            float bv = -INFINITY;
            for (int g = 0; g < groups; ++g)
                if (strength[g] != INFINITY && (best < 0 || strength[g] > bv)) { best = g; bv = strength[g]; }
            if (best >= 0) strength[best] = INFINITY;      // kept
        }
        for (int g = 0; g < groups; ++g)
            if (strength[g] != INFINITY)
                for (int i = 0; i < per; ++i) pick[g * per + i] = -INFINITY;
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float bv = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (pick[e] > bv) { best = e; bv = pick[e]; }
        if (best < 0) best = 0;                            // cannot happen: top never exceeds the experts in the race
        pick[best] = -INFINITY;
        chosen[(size_t)r * top + k] = best;
        weights[(size_t)r * top + k] = sc[best];
        total += sc[best];
    }
    const float inv = 1.f / (total + weight_eps);
    for (int k = 0; k < top; ++k) weights[(size_t)r * top + k] *= inv;
}

// ------------------------------------------------------------------------------------------------------------
// hidden[r * top + k][j] = silu(Wg[e][j] . x[r]) * (Wu[e][j] . x[r]),  e = chosen[r][k];  w_gu (E, 2, F, d).
// A CTA per (row and choice, block of COLS hidden columns); a warp a column at a time.
// ------------------------------------------------------------------------------------------------------------
constexpr int MOE_COLS = 32;

template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gate_up_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ chosen, const T* __restrict__ w_gu,
                   T* __restrict__ hidden, int d, int top, int E, int F) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    const int pair = blockIdx.x, r = pair / top;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    const int e = chosen[pair];
    if (e < 0 || e >= E) return;
    for (int i = tid; i < d; i += blockDim.x) smem[i] = to_f32(x[(size_t)r * ldx + i]);
    __syncthreads();
    const bool vec = d % Vec16<T>::N == 0 && ((uintptr_t)w_gu % 16 == 0);
    const T* wg = w_gu + (size_t)e * 2 * F * d;
    const T* wu = wg + (size_t)F * d;
    const int j_end = min(F, (int)(blockIdx.y + 1) * MOE_COLS);
    for (int j = blockIdx.y * MOE_COLS + warp; j < j_end; j += nw) {
        const float g = warp_dot<T>(wg + (size_t)j * d, smem, d, lane, vec);
        const float u = warp_dot<T>(wu + (size_t)j * d, smem, d, lane, vec);
        if (lane == 0) hidden[(size_t)pair * F + j] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

// ------------------------------------------------------------------------------------------------------------
// out[r][c] = sum_k weights[r][k] * (Wd[e_k][c] . hidden[r * top + k])  (+ shared_gate[r] * shared[r][c]);
// w_down (E, d, F).  A CTA per (row, block of COLS output columns).
// ------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(MOE_THREADS)
moe_down_kernel(const T* __restrict__ hidden, const int* __restrict__ chosen, const float* __restrict__ weights,
                const T* __restrict__ w_down, const T* __restrict__ shared, int lds,
                const float* __restrict__ shared_gate, T* __restrict__ out, int d, int top, int E, int F) {
    extern __shared__ float smem[];                // [top][F]
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nw = blockDim.x >> 5;
    pdl_wait();
    for (int i = tid; i < top * F; i += blockDim.x) smem[i] = to_f32(hidden[(size_t)r * top * F + i]);
    __syncthreads();
    const bool vec = F % Vec16<T>::N == 0 && ((uintptr_t)w_down % 16 == 0);
    const float sg = shared != nullptr ? (shared_gate != nullptr ? shared_gate[r] : 1.f) : 0.f;
    const int c_end = min(d, (int)(blockIdx.y + 1) * MOE_COLS);
    for (int c = blockIdx.y * MOE_COLS + warp; c < c_end; c += nw) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int e = chosen[(size_t)r * top + k];
            if (e < 0 || e >= E) continue;
            const float v = warp_dot<T>(w_down + ((size_t)e * d + c) * F, smem + (size_t)k * F, F, lane, vec);
            acc = fmaf(weights[(size_t)r * top + k], v, acc);
        }
        if (lane == 0) {
            if (shared != nullptr) acc = fmaf(sg, to_f32(shared[(size_t)r * lds + c]), acc);
            out[(size_t)r * d + c] = from_f32<T>(acc);
        }
    }
}

template <typename K>
int set_smem(K kernel, size_t bytes, const char* what) {
    if (bytes > 200 * 1024) {
        tis_set_error("%s: %zu bytes of shared memory a CTA (at most 200 KB)", what, bytes);
        return TIS_BAD_SIZE;
    }
    if (bytes > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    return TIS_OK;
}

}  // namespace

TIS_API int tis_moe_route(int dtype, const void* x, int ldx, const float* wr, const float* corr, const float* w_sg,
                          int n, int d, int E, int groups, int keep, int top, float weight_eps, int* chosen,
                          float* weights, float* shared_gate, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || E <= 0 || top <= 0 || top > E || groups < 0 || (groups > 0 && (E % groups || keep <= 0 || keep > groups ||
        top > E / groups * keep)) || (w_sg != nullptr && shared_gate == nullptr)) {
        tis_set_error("moe_route: %d experts, top %d, %d groups of which %d kept", E, top, groups, keep);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * ((size_t)d + 2 * (size_t)E + (size_t)(groups > 0 ? groups : 1));
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_route_kernel<T>, smem, "moe_route");
        if (st != TIS_OK) return st;
        tis_launch(moe_route_kernel<T>, dim3(n), dim3(MOE_THREADS), smem, stream, (const T*)x, ldx, wr, corr, w_sg, d, E,
                   groups, keep, top, weight_eps, chosen, weights, shared_gate);
    });
    return tis_check_launch("moe_route");
}

TIS_API int tis_moe_gate_up(int dtype, const void* x, int ldx, const int* chosen, const void* w_gu, void* hidden, int n,
                            int d, int top, int E, int F, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || top <= 0 || E <= 0 || F <= 0) {
        tis_set_error("moe_gate_up: width %d, top %d, %d experts of %d hidden", d, top, E, F);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * (size_t)d;
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_gate_up_kernel<T>, smem, "moe_gate_up");
        if (st != TIS_OK) return st;
        tis_launch(moe_gate_up_kernel<T>, dim3(n * top, (F + MOE_COLS - 1) / MOE_COLS), dim3(MOE_THREADS), smem, stream,
                   (const T*)x, ldx, chosen, (const T*)w_gu, (T*)hidden, d, top, E, F);
    });
    return tis_check_launch("moe_gate_up");
}

TIS_API int tis_moe_down(int dtype, const void* hidden, const int* chosen, const float* weights, const void* w_down,
                         const void* shared, int lds, const float* shared_gate, void* out, int n, int d, int top, int E,
                         int F, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (d <= 0 || top <= 0 || E <= 0 || F <= 0) {
        tis_set_error("moe_down: width %d, top %d, %d experts of %d hidden", d, top, E, F);
        return TIS_BAD_SIZE;
    }
    const size_t smem = sizeof(float) * (size_t)top * F;
    TIS_DISPATCH_DTYPE(dtype, T, {
        const int st = set_smem(moe_down_kernel<T>, smem, "moe_down");
        if (st != TIS_OK) return st;
        tis_launch(moe_down_kernel<T>, dim3(n, (d + MOE_COLS - 1) / MOE_COLS), dim3(MOE_THREADS), smem, stream,
                   (const T*)hidden, chosen, weights, (const T*)w_down, (const T*)shared, lds, shared_gate, (T*)out, d, top,
                   E, F);
    });
    return tis_check_launch("moe_down");
}
