// Mixture of experts: the router's choice, the experts' products for (token, chosen expert) pairs, the gated unit
// with a capped gate, and the weighted sum.
//
// A step's tokens each choose `top` of E experts.  Pair i = t * top + k is token t's k-th choice (in the order of
// falling score); expert_of[i] names its expert, weight[i] its share.  Everything is worked out on the device from
// the router's logits, with grids that depend on the number of tokens only, so a step can be captured in a graph.
#include "common.cuh"

// ---------------------------------------------------------------- the router's choice
// One warp a token.  s = softmax(z) over all experts (float32).  With groups > 1 the experts form `groups` equal
// runs of neighbours, a group's score is its largest s, and only experts of the `keep` best groups can be chosen.
// The `top` largest s among those are chosen (the lower index on a tie); weight = s / (sum of the chosen s + tiny).
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ldz, int* __restrict__ expert_of, float* __restrict__ weight, int T, int E,
                 int top, int groups, int keep, float tiny) {
    extern __shared__ float route_smem[];                 // per warp: E scores, then `groups` group scores
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T) return;
    float* s = route_smem + (size_t)warp * (E + groups);
    float* gs = s + E;
    const float* zr = z + (size_t)t * ldz;
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) {
        const float v = expf(zr[e] - m);
        s[e] = v;
        sum += v;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < E; e += 32) s[e] *= inv;
    __syncwarp();
    const int gsize = E / groups;
    if (groups > 1) {
        for (int g = lane; g < groups; g += 32) {
            float b = -1.f;
            for (int e = g * gsize; e < (g + 1) * gsize; ++e) b = fmaxf(b, s[e]);
            gs[g] = b;
        }
        __syncwarp();
        for (int r = 0; r < keep; ++r) {                  // the best group not yet kept becomes -2: kept
            float bv = -1.f;
            int bi = 0x7fffffff;
            for (int g = lane; g < groups; g += 32)
                if (gs[g] > bv) { bv = gs[g]; bi = g; }
            warp_argmax(bv, bi);
            __syncwarp();
            if (lane == 0 && bi < groups) gs[bi] = -2.f;
            __syncwarp();
        }
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float bv = -1.f;
        int bi = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const bool open = groups <= 1 || gs[e / gsize] == -2.f;
            if (open && s[e] > bv) { bv = s[e]; bi = e; }
        }
        warp_argmax(bv, bi);
        __syncwarp();
        if (lane == 0) {
            expert_of[(size_t)t * top + k] = bi < E ? bi : 0;
            weight[(size_t)t * top + k] = bv;             // the score for now; divided below
            if (bi < E) s[bi] = -1.f;
        }
        total += bv;
        __syncwarp();
    }
    const float scale = 1.0f / (total + tiny);
    __syncwarp();
    for (int k = lane; k < top; k += 32) weight[(size_t)t * top + k] *= scale;
}

RB_EXPORT int rb_moe_route(const float* z, int ldz, int* expert_of, float* weight, int T, int E, int top, int groups, int keep,
                           float tiny, cudaStream_t st) {
    if (T <= 0) return 0;
    if (groups < 1 || E % groups || top < 1 || top > E || keep < 1 || keep > groups || (long long)keep * (E / groups) < top)
        return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)4 * (E + groups) * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(moe_route_kernel, dim3((T + 3) / 4), dim3(128), smem, st, z, ldz, expert_of, weight, T, E, top,
                         groups, keep, tiny);
}

// ---------------------------------------------------------------- a pair's product, weights streamed
// out[i, n] = sum_k x[i / in_div, k] * W[expert_of[i]][n, k] for every pair i: the form for few pairs (decoded tokens)
// and the float32 path.  One CTA takes one pair and a run of output rows; a warp an output row at a time, the lanes
// striding k, so every sum has one order whatever else the step holds.  W: [E, N, K] contiguous.
template <typename TA, typename TO>
__global__ void __launch_bounds__(256)
moe_pair_linear_kernel(const TA* __restrict__ x, int ldx, int in_div, const TA* __restrict__ W, const int* __restrict__ expert_of,
                       TO* __restrict__ out, int ldo, int N, int K, int rows_per_cta) {
    extern __shared__ float xs[];                         // K floats
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const TA* xr = x + (size_t)(i / in_div) * ldx;
    for (int k = threadIdx.x; k < K; k += blockDim.x) xs[k] = to_f32(xr[k]);
    __syncthreads();
    const TA* We = W + (size_t)expert_of[i] * N * K;
    const int n0 = blockIdx.y * rows_per_cta;
    const int n1 = min(N, n0 + rows_per_cta);
    for (int n = n0 + warp; n < n1; n += nwarps) {
        const TA* wr = We + (size_t)n * K;
        float acc = 0.f;
        for (int k = lane; k < K; k += 32) acc = fmaf(xs[k], to_f32(wr[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) out[(size_t)i * ldo + n] = from_f32<TO>(acc);
    }
}

RB_EXPORT int rb_moe_pair_linear(const void* x, int ldx, int in_div, const void* W, const int* expert_of, void* out, int ldo,
                                 int act_dtype, int pairs, int N, int K, cudaStream_t st) {
    if (pairs <= 0 || N <= 0) return 0;
    const int rows_per_cta = 64;
    dim3 grid(pairs, (N + rows_per_cta - 1) / rows_per_cta);
    const size_t smem = (size_t)K * sizeof(float);
    if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(moe_pair_linear_kernel<float, float>, grid, dim3(256), smem, st, (const float*)x, ldx, in_div,
                             (const float*)W, expert_of, (float*)out, ldo, N, K, rows_per_cta);
    return rb_launch_pdl(moe_pair_linear_kernel<bf16, bf16>, grid, dim3(256), smem, st, (const bf16*)x, ldx, in_div,
                         (const bf16*)W, expert_of, (bf16*)out, ldo, N, K, rows_per_cta);
}

// ---------------------------------------------------------------- the gated unit with a capped gate
// in[r] = [gate (F numbers) | up (F numbers)];  g = min(gate, limit), u = clamp(up, -limit, limit);
// out[r, f] = g * sigmoid(alpha * g) * (u + 1).  float32 arithmetic, one rounding at the store.
template <typename TA>
__global__ void clamped_glu_kernel(const TA* __restrict__ in, int ldi, TA* __restrict__ out, int ldo, int F, float limit,
                                   float alpha, long long total) {
    pdl_launch_dependents();
    pdl_wait();
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        const long long r = e / F;
        const int f = (int)(e % F);
        const float g = fminf(to_f32(in[r * ldi + f]), limit);
        const float u = fminf(fmaxf(to_f32(in[r * ldi + F + f]), -limit), limit);
        out[r * ldo + f] = from_f32<TA>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
    }
}

RB_EXPORT int rb_clamped_glu(const void* in, int ldi, void* out, int ldo, int act_dtype, int rows, int F, float limit,
                             float alpha, cudaStream_t st) {
    const long long total = (long long)rows * F;
    if (total <= 0) return 0;
    const int blocks = (int)min((long long)4096, (total + 255) / 256);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(clamped_glu_kernel<float>, dim3(blocks), dim3(256), 0, st, (const float*)in, ldi, (float*)out, ldo, F,
                             limit, alpha, total);
    return rb_launch_pdl(clamped_glu_kernel<bf16>, dim3(blocks), dim3(256), 0, st, (const bf16*)in, ldi, (bf16*)out, ldo, F, limit,
                         alpha, total);
}

// ---------------------------------------------------------------- the weighted sum of a token's experts
// out[t, :] = sum_k weight[t, k] * y[row_of ? row_of[t * top + k] : t * top + k, :]  (+ shared[t, :]), k ascending, float32
// sums.  row_of: where a pair's row lies when the pairs were put in the order of their experts.
template <typename TA>
__global__ void moe_combine_kernel(const TA* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ weight,
                                   const TA* __restrict__ shared, TA* __restrict__ out, int H, int top) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int k = 0; k < top; ++k) {
            const int pair = t * top + k;
            const size_t row = row_of ? (size_t)row_of[pair] : (size_t)pair;
            acc = fmaf(weight[pair], to_f32(y[row * H + i]), acc);
        }
        if (shared != nullptr) acc += to_f32(shared[(size_t)t * H + i]);
        out[(size_t)t * H + i] = from_f32<TA>(acc);
    }
}

RB_EXPORT int rb_moe_combine(const void* y, const int* row_of, const float* weight, const void* shared, void* out,
                             int act_dtype, int T, int H, int top, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(moe_combine_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)y, row_of, weight,
                             (const float*)shared, (float*)out, H, top);
    return rb_launch_pdl(moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, st, (const bf16*)y, row_of, weight,
                         (const bf16*)shared, (bf16*)out, H, top);
}
