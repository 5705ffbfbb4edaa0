// Attention over a paged cache of latents: every token leaves one vector [rank + rot] in the cache (a normed
// latent of `rank` numbers, then a rotated key part of `rot` numbers that all heads share), and the heads' keys
// and values are linear maps of the latent.  The maps are folded into the query and the output: with
// k_h = U_h c and v_h = V_h c,
//     q_h . k_h = (U_h^T q_h) . c        and        sum_j a_j v_h(j) = V_h (sum_j a_j c_j),
// so a head scores the cached latents with a query of `rank` numbers (plus the rotated part against the shared
// rotated key) and averages the latents themselves; one cached vector serves every head, as key and as value.
//
// Kernels: the write of a step's latents (norm, rotation, page write, rotation of the queries' rotated parts),
// the attention itself on the CUDA cores for any sizes and element types (float32 path, and the plain twin of
// the tensor-core kernels, which are the engine's paged attention kernels run with one shared key/value head whose
// keys and values are both the cached vector), the heads' output gate, and the float32 products head by head.
#include "common.cuh"

#define LAT_MAX_RANK 1024

// ---------------------------------------------------------------- write of a step's latents
// One CTA a token.  x: the token's row of the in-projection; the latent's raw numbers at column c_off (rank of
// them, normed here with weight w), the shared key part behind them (rot numbers, rotated here; element i pairs
// with i + rot/2).  Both go to the page of the token's position: pool [pages, page_size, width], width >= rank + rot
// (a multiple of 16 for the tensor-core kernels; the columns behind rank + rot are written as zeros).
// The rotated parts of the queries (q at column q_off of xq, heads of [dim | rot]) are rotated into the query rows
// that the attention reads, q_abs [T, heads, width], at columns [rank, rank + rot) of a head; the columns behind are
// zeroed; the first `rank` columns are another kernel's.  cos, sin: float32 [positions, rot/2].
template <typename TA>
__global__ void latent_write_kernel(const TA* __restrict__ x, int ldx, int c_off, const void* __restrict__ w, int w_dtype,
                                    float eps, int rank, int rot, const float* __restrict__ cosT,
                                    const float* __restrict__ sinT, const int* __restrict__ pos,
                                    const int* __restrict__ tok_seg, const int* __restrict__ block_table, int bt_stride,
                                    int page_size, TA* __restrict__ pool, int width, int write_cache,
                                    const TA* __restrict__ xq, int ldq, int q_off, int heads, int dim,
                                    TA* __restrict__ q_abs) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int p = pos[t];
    const int half = rot >> 1;
    const float* cr = cosT + (size_t)p * half;
    const float* sr = sinT + (size_t)p * half;
    if (write_cache) {
        const TA* src = x + (size_t)t * ldx + c_off;
        float ss = 0.f;
        for (int i = threadIdx.x; i < rank; i += blockDim.x) {
            const float v = to_f32(src[i]);
            ss += v * v;
        }
        ss = block_sum(ss, scratch);
        const float rstd = 1.0f / sqrtf(ss / (float)rank + eps);
        const int page = block_table[(size_t)tok_seg[t] * bt_stride + p / page_size];
        if (page >= 0) {
            TA* dst = pool + ((size_t)page * page_size + (p % page_size)) * (size_t)width;
            for (int i = threadIdx.x; i < rank; i += blockDim.x)
                dst[i] = from_f32<TA>(to_f32(src[i]) * rstd * load_as_f32(w, w_dtype, i));
            for (int i = threadIdx.x; i < half; i += blockDim.x) {
                const float u = to_f32(src[rank + i]), v = to_f32(src[rank + half + i]);
                dst[rank + i] = from_f32<TA>(u * cr[i] - v * sr[i]);
                dst[rank + half + i] = from_f32<TA>(v * cr[i] + u * sr[i]);
            }
            for (int i = rank + rot + threadIdx.x; i < width; i += blockDim.x) dst[i] = from_f32<TA>(0.f);
        }
    }
    if (q_abs != nullptr) {
        TA* qa = q_abs + (size_t)t * heads * width;
        for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
            const int h = e / half, i = e % half;
            const TA* qh = xq + (size_t)t * ldq + q_off + (size_t)h * (dim + rot) + dim;
            const float u = to_f32(qh[i]), v = to_f32(qh[half + i]);
            TA* dst = qa + (size_t)h * width + rank;
            dst[i] = from_f32<TA>(u * cr[i] - v * sr[i]);
            dst[half + i] = from_f32<TA>(v * cr[i] + u * sr[i]);
        }
        const int pad = width - rank - rot;
        for (int e = threadIdx.x; e < heads * pad; e += blockDim.x)
            qa[(size_t)(e / pad) * width + rank + rot + e % pad] = from_f32<TA>(0.f);
    }
}

RB_EXPORT int rb_latent_write(const void* x, int ldx, int c_off, const void* w, int w_dtype, float eps, int rank, int rot,
                              const float* cosT, const float* sinT, const int* pos, const int* tok_seg,
                              const int* block_table, int bt_stride, int page_size, void* pool, int width, int write_cache,
                              const void* xq, int ldq, int q_off, int heads, int dim, void* q_abs, int act_dtype, int T,
                              cudaStream_t st) {
    if (T <= 0) return 0;
    if ((rot & 1) || width < rank + rot) return (int)cudaErrorInvalidValue;
    const int threads = rank >= 512 ? 256 : 128;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(latent_write_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)x, ldx, c_off, w, w_dtype,
                             eps, rank, rot, cosT, sinT, pos, tok_seg, block_table, bt_stride, page_size, (float*)pool, width,
                             write_cache, (const float*)xq, ldq, q_off, heads, dim, (float*)q_abs);
    return rb_launch_pdl(latent_write_kernel<bf16>, dim3(T), dim3(threads), 0, st, (const bf16*)x, ldx, c_off, w, w_dtype, eps,
                         rank, rot, cosT, sinT, pos, tok_seg, block_table, bt_stride, page_size, (bf16*)pool, width, write_cache,
                         (const bf16*)xq, ldq, q_off, heads, dim, (bf16*)q_abs);
}

// ---------------------------------------------------------------- attention on the CUDA cores
// One warp owns one (token, head).  Keys are taken in tiles of 32 aligned to absolute positions, lane j of a tile
// scores key j against the whole cached vector, and the online softmax (float32) advances tile by tile; the
// accumulator over the latent's `rank` numbers is spread over the lanes.  A row looks at nothing but its own keys
// and the tiles are fixed by position, so a token's result does not depend on how the prompt was cut or on what
// else is in the batch.  q_abs [T, heads, width] (a head's query in the latent's space, then its rotated part),
// out [T, heads, width] (the first `rank` columns of a head are written).
// A key at position j is visible to the query at p iff lo <= j <= p, lo = max(0, p - window + 1) for window > 0.
// sink (float32 [heads] or null): a term exp(sink_h) in the denominator that has no key and no value.
template <typename TA>
__global__ void __launch_bounds__(128)
latent_attention_simt_kernel(const TA* __restrict__ q_abs, const TA* __restrict__ pool,
                             const int* __restrict__ pos, const int* __restrict__ tok_seg,
                             const int* __restrict__ block_table, int bt_stride, int page_size,
                             const float* __restrict__ sink, TA* __restrict__ out, int heads, int rank, int rot, int width,
                             float scale, int window) {
    extern __shared__ float qs_all[];                    // 4 warps x (rank + rot) floats
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * 4 + warp;
    if (h >= heads) return;                              // no block-wide barrier below
    const int W = rank + rot;
    const int p = pos[t];
    const int* bt = block_table + (size_t)tok_seg[t] * bt_stride;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    float* qs = qs_all + warp * W;
    const TA* ql = q_abs + ((size_t)t * heads + h) * width;
    for (int d = lane; d < W; d += 32) qs[d] = to_f32(ql[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[LAT_MAX_RANK / 32];
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] = 0.f;

    for (int j0 = (lo / 32) * 32; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= p;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0) {
                s = __int_as_float(0x7fc00000);          // a page that was given back: show it as NaN
            } else {
                const TA* kr = pool + ((size_t)page * page_size + (j % page_size)) * (size_t)width;
                float dot = 0.f;
                for (int d = 0; d < W; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pj = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);             // m = -inf on the first tile gives 0
        l = l * alpha + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] *= alpha;
        const int jend = min(32, p - j0 + 1);
        for (int jj = max(0, lo - j0); jj < jend; ++jj) {
            const float pjj = __shfl_sync(0xffffffffu, pj, jj);
            const int jk = j0 + jj;
            const int page = bt[jk / page_size];
            if (page < 0) continue;
            const TA* vr = pool + ((size_t)page * page_size + (jk % page_size)) * (size_t)width;
#pragma unroll
            for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < rank) acc[i] = fmaf(pjj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    if (sink != nullptr) {
        const float sk = sink[h];
        const float m_new = fmaxf(m, sk);
        const float alpha = expf(m - m_new);
        l = l * alpha + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < LAT_MAX_RANK / 32; ++i) acc[i] *= alpha;
    }
    TA* orow = out + ((size_t)t * heads + h) * width;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < LAT_MAX_RANK / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) orow[d] = from_f32<TA>(acc[i] * inv);
    }
}

RB_EXPORT int rb_latent_attention_simt(const void* q_abs, const void* pool, const int* pos,
                                       const int* tok_seg, const int* block_table, int bt_stride, int page_size,
                                       const float* sink, void* out, int act_dtype, int T, int heads, int rank, int rot,
                                       int width, float scale, int window, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rank <= 0 || rank > LAT_MAX_RANK || heads <= 0 || width < rank + rot) return (int)cudaErrorInvalidValue;
    dim3 grid(T, (heads + 3) / 4);
    const size_t smem = (size_t)4 * (rank + rot) * sizeof(float);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(latent_attention_simt_kernel<float>, grid, dim3(128), smem, st, (const float*)q_abs,
                             (const float*)pool, pos, tok_seg, block_table, bt_stride, page_size, sink,
                             (float*)out, heads, rank, rot, width, scale, window);
    return rb_launch_pdl(latent_attention_simt_kernel<bf16>, grid, dim3(128), smem, st, (const bf16*)q_abs,
                         (const bf16*)pool, pos, tok_seg, block_table, bt_stride, page_size, sink, (bf16*)out, heads,
                         rank, rot, width, scale, window);
}

// ---------------------------------------------------------------- the output gate of the heads
// x[t, h * vdim + e] *= sigmoid(gate[t * ldg + h]), in place.  The gate's logistic is float32.
template <typename TA>
__global__ void head_gate_kernel(TA* __restrict__ x, const TA* __restrict__ gate, int ldg, int heads, int vdim) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    for (int e = threadIdx.x; e < heads * vdim; e += blockDim.x) {
        const float g = 1.0f / (1.0f + expf(-to_f32(gate[(size_t)t * ldg + e / vdim])));
        TA* p = x + (size_t)t * heads * vdim + e;
        *p = from_f32<TA>(to_f32(*p) * g);
    }
}

RB_EXPORT int rb_head_gate(void* x, const void* gate, int ldg, int act_dtype, int T, int heads, int vdim, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = heads * vdim >= 1024 ? 256 : 128;
    if (act_dtype == RB_F32)
        return rb_launch_pdl(head_gate_kernel<float>, dim3(T), dim3(threads), 0, st, (float*)x, (const float*)gate, ldg, heads, vdim);
    return rb_launch_pdl(head_gate_kernel<bf16>, dim3(T), dim3(threads), 0, st, (bf16*)x, (const bf16*)gate, ldg, heads, vdim);
}

// ---------------------------------------------------------------- float32 products head by head
// C[b][m, n] = sum_k A[b][m, k] * W[b][n, k] for b < batch, in true float32 (FFMA), every element accumulated over
// k in ascending order by one thread: the 32-bit path's form of the two folded maps.  Strides in elements.
#define HB_BM 64
#define HB_BN 64
#define HB_BK 16

__global__ void __launch_bounds__(256)
gemm_f32_heads_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M, int N, int K,
                      int lda, int ldw, int ldc, long long sa, long long sw, long long sc) {
    __shared__ float As[HB_BK][HB_BM + 4];
    __shared__ float Ws[HB_BK][HB_BN + 4];
    pdl_launch_dependents();
    pdl_wait();
    A += (size_t)blockIdx.z * sa;
    W += (size_t)blockIdx.z * sw;
    C += (size_t)blockIdx.z * sc;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int m0 = blockIdx.y * HB_BM, n0 = blockIdx.x * HB_BN;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += HB_BK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int e = tid + r * 256;
            const int row = e >> 4, kk = e & 15;
            const int k = k0 + kk;
            const int m = m0 + row, n = n0 + row;
            As[kk][row] = (m < M && k < K) ? A[(size_t)m * lda + k] : 0.f;
            Ws[kk][row] = (n < N && k < K) ? W[(size_t)n * ldw + k] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HB_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(size_t)m * ldc + n] = acc[i][j];
        }
    }
}

RB_EXPORT int rb_gemm_f32_heads(const float* A, const float* W, float* C, int batch, int M, int N, int K, int lda, int ldw,
                                int ldc, long long sa, long long sw, long long sc, cudaStream_t st) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    dim3 grid((N + HB_BN - 1) / HB_BN, (M + HB_BM - 1) / HB_BM, batch);
    return rb_launch_pdl(gemm_f32_heads_kernel, grid, dim3(256), 0, st, A, W, C, M, N, K, lda, ldw, ldc, sa, sw, sc);
}

// ---------------------------------------------------------------- a prompt's keys and values, expanded per head
// A long portion of a prompt is cheaper with the heads' keys and values written out (a head then scores dim + rot
// numbers a key and averages vdim, not twice the cached vector's width): the visible latents are gathered, carried
// through [U; V] by one product, and scattered here into scratch pools [pages, heads, page_size, head] that the
// paged tensor-core attention reads with the request's own block table.  Key of head h: [U_h c | rotated part | 0],
// value: [V_h c | 0].  slot = page * page_size + row, one per gathered latent.
__global__ void latent_expand_scatter_kernel(const bf16* __restrict__ kv, int ldkv, const bf16* __restrict__ lat, int ldl,
                                             int rank, int rot, const int* __restrict__ slots, int page_size,
                                             bf16* __restrict__ kx, bf16* __restrict__ vx, int heads, int dim, int vdim,
                                             int head) {
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x;
    const int slot = slots[i];
    const int page = slot / page_size, row = slot - page * page_size;
    const bf16* kvr = kv + (size_t)i * ldkv;
    const bf16* lr = lat + (size_t)i * ldl + rank;
    const bf16 zero = __float2bfloat16_rn(0.f);
    for (int e = threadIdx.x; e < heads * head; e += blockDim.x) {
        const int h = e / head, d = e - h * head;
        const size_t at = (((size_t)page * heads + h) * page_size + row) * head + d;
        kx[at] = d < dim ? kvr[h * dim + d] : (d < dim + rot ? lr[d - dim] : zero);
        vx[at] = d < vdim ? kvr[heads * dim + h * vdim + d] : zero;
    }
}

RB_EXPORT int rb_latent_expand_scatter(const void* kv, int ldkv, const void* lat, int ldl, int rank, int rot, const int* slots,
                                       int page_size, void* kx, void* vx, int heads, int dim, int vdim, int head, int n,
                                       cudaStream_t st) {
    if (n <= 0) return 0;
    if (head < dim + rot || head < vdim) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(latent_expand_scatter_kernel, dim3(n), dim3(256), 0, st, (const bf16*)kv, ldkv, (const bf16*)lat, ldl,
                         rank, rot, slots, page_size, (bf16*)kx, (bf16*)vx, heads, dim, vdim, head);
}

// The queries of the expanded form: head h of token t is [its unrotated part | its rotated part, already turned (it
// lies in the folded query row behind the latent's columns) | 0].
__global__ void latent_expand_query_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ q_abs, int width,
                                           int rank, bf16* __restrict__ qx, int heads, int dim, int rot, int head) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const bf16 zero = __float2bfloat16_rn(0.f);
    for (int e = threadIdx.x; e < heads * head; e += blockDim.x) {
        const int h = e / head, d = e - h * head;
        qx[(size_t)t * heads * head + e] = d < dim ? q[(size_t)t * ldq + (size_t)h * (dim + rot) + d]
                                           : (d < dim + rot ? q_abs[((size_t)t * heads + h) * width + rank + d - dim] : zero);
    }
}

RB_EXPORT int rb_latent_expand_query(const void* q, int ldq, const void* q_abs, int width, int rank, void* qx, int heads,
                                     int dim, int rot, int head, int T, cudaStream_t st) {
    if (T <= 0) return 0;
    return rb_launch_pdl(latent_expand_query_kernel, dim3(T), dim3(256), 0, st, (const bf16*)q, ldq, (const bf16*)q_abs, width,
                         rank, (bf16*)qx, heads, dim, rot, head);
}

// The values of the tokens that ran in the expanded form (segments of several tokens) into the rows that the output
// projection reads: out[t, h * vdim + e] = ox[t, h * head + e]; rows of single tokens are another kernel's.
__global__ void latent_take_values_kernel(const bf16* __restrict__ ox, const int* __restrict__ tok_seg,
                                          const int* __restrict__ cu_q, bf16* __restrict__ out, int heads, int vdim, int head) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seg = tok_seg[t];
    if (cu_q[seg + 1] - cu_q[seg] <= 1) return;
    for (int e = threadIdx.x; e < heads * vdim; e += blockDim.x) {
        const int h = e / vdim, d = e - h * vdim;
        out[(size_t)t * heads * vdim + e] = ox[((size_t)t * heads + h) * head + d];
    }
}

RB_EXPORT int rb_latent_take_values(const void* ox, const int* tok_seg, const int* cu_q, void* out, int heads, int vdim,
                                    int head, int T, cudaStream_t st) {
    if (T <= 0) return 0;
    return rb_launch_pdl(latent_take_values_kernel, dim3(T), dim3(256), 0, st, (const bf16*)ox, tok_seg, cu_q, (bf16*)out, heads,
                         vdim, head);
}

// out[i, :] = x[index[i], :] for rows of `bytes` bytes (a multiple of 16), 16 bytes a thread and step.
__global__ void latent_gather_rows_kernel(const unsigned char* __restrict__ x, long long ldx_bytes, const int* __restrict__ index,
                                          unsigned char* __restrict__ out, int bytes) {
    pdl_launch_dependents();
    pdl_wait();
    const unsigned char* src = x + (size_t)index[blockIdx.x] * ldx_bytes;
    unsigned char* dst = out + (size_t)blockIdx.x * bytes;
    for (int b = threadIdx.x * 16; b < bytes; b += blockDim.x * 16)
        *reinterpret_cast<uint4*>(dst + b) = *reinterpret_cast<const uint4*>(src + b);
}

RB_EXPORT int rb_latent_gather_rows(const void* x, long long ldx_bytes, const int* index, void* out, int bytes, int n,
                                    cudaStream_t st) {
    if (n <= 0) return 0;
    if (bytes % 16 || ldx_bytes % 16 || ((uintptr_t)x % 16) || ((uintptr_t)out % 16)) return (int)cudaErrorInvalidValue;
    return rb_launch_pdl(latent_gather_rows_kernel, dim3(n), dim3(64), 0, st, (const unsigned char*)x, ldx_bytes, index,
                         (unsigned char*)out, bytes);
}
