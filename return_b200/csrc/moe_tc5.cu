// The experts' products of a prompt on the fifth-generation tensor cores: C[place, n] = sum_k A[place, k] W[e][n, k]
// over the (token, expert) pairs in the order of their experts (A holds their rows in that order), bfloat16 with
// float32 accumulation in tensor memory, operands by TMA.
//
// The kernel is the persistent product kernel of gemm_tc5.cu (a producer thread, an MMA thread, four epilogue warps,
// a ring of operand stages, two accumulators in tensor memory) with another list of tiles: an expert's run of places
// is cut into tiles of 128 rows that begin where the run begins, so a tile never mixes experts; the rows of a tile
// behind the run's end belong to the next expert (or lie behind the matrix and come as zeros) and are computed but
// not stored.  The weights of all experts are one matrix [E * N, K]; a tile's box of 256 weight rows begins at its
// expert's n-th row and may reach into the next expert's rows, whose columns are not stored either.  How many tiles
// there are follows from the router's choice, which only the device knows: every CTA works the list out from the
// offsets of the runs, and the grid is as large as the SMs or the worst case, whichever is smaller.
//
// Every mbarrier wait is bounded; a wait that gives up raises *status and the kernel still frees its tensor memory.
#include <cuda.h>

#include "tc5.cuh"
#include "tma.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128;
constexpr int BK = 64;                    // bf16 elements: one 128-byte swizzle row
constexpr int BN = 256;
constexpr int STAGES = 4;
constexpr int THREADS = 192;              // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue
constexpr int MAX_EXPERTS = 1024;

struct Tile {
    int m0;        // first place (row of A and of C)
    int rows;      // places of the tile that belong to its expert
    int w_row;     // first row of the tile in the matrix of all experts' weights
    int n0;        // first output column
};

// Tiles are numbered with the row tiles of all experts fastest, so that neighbours share a block of weights only
// within an expert but the tokens' rows stay in L2 across the output columns.
__device__ __forceinline__ Tile locate(const int* s_start, const int* s_off, int E, int N, int total_m, int tile) {
    const int nt = tile / total_m, r = tile - nt * total_m;
    int lo = 0, hi = E;                                     // the last expert whose first tile is not behind r
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (s_start[mid] <= r) lo = mid; else hi = mid;
    }
    const int mt = r - s_start[lo];
    Tile t;
    t.m0 = s_off[lo] + mt * BM;
    t.rows = min(BM, s_off[lo + 1] - t.m0);
    t.n0 = nt * BN;
    t.w_row = lo * N + t.n0;
    return t;
}

__device__ __forceinline__ void store_chunk(bf16* dst, const unsigned (&r)[32], int n_valid) {
    if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
            v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
            *reinterpret_cast<uint4*>(dst + j) = v;
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j)
        if (j < n_valid) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
}

__global__ void __launch_bounds__(THREADS)
moe_tc5_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               const int* __restrict__ offsets, int E, bf16* __restrict__ out, int N, int K, int ldo,
               int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr unsigned A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_slot;
    __shared__ int s_start[MAX_EXPERTS + 1], s_off[MAX_EXPERTS + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr unsigned TMEM_COLS = 2 * BN;
    const int nkb = (K + BK - 1) / BK;                      // k blocks past K are zero-filled by the copy

    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) {
        tma::prefetch_desc(&map_a);
        tma::prefetch_desc(&map_w);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
#pragma unroll
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 4); }
        mbar_init_fence();
    }
    pdl_wait();                                             // the offsets and the rows come from the kernels before
    for (int e = tid; e <= E; e += THREADS) s_off[e] = offsets[e];
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    if (tid == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            s_start[e] = run;
            run += (s_off[e + 1] - s_off[e] + BM - 1) / BM;
        }
        s_start[E] = run;
    }
    __syncthreads();
    const int total_m = s_start[E];
    const int tiles = total_m * ((N + BN - 1) / BN);
    const unsigned tacc = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                    // ---- producer
            int it = 0;                                     // k blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const Tile t = locate(s_start, s_off, E, N, total_m, tile);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1) && ok;
                    const unsigned full = smem_u32(&full_bar[s]);
                    mbar_arrive_expect_tx(full, STAGE_BYTES);
                    const unsigned dst = smem_u32(base + (size_t)s * STAGE_BYTES);
                    tma::load_2d(dst, &map_a, kb * BK, t.m0, full);
                    tma::load_2d(dst + A_BYTES, &map_w, kb * BK, t.w_row, full);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                    // ---- MMA issuer
            const unsigned idesc = instr_desc_bf16(BM, BN);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(smem_u32(&acc_empty[buf]), ((local >> 1) - 1) & 1) && ok;
                fence_after_sync();
                const unsigned d = tacc + buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1) && ok;
                    fence_after_sync();
                    const unsigned a = smem_u32(base + (size_t)s * STAGE_BYTES), b = a + A_BYTES;
#pragma unroll
                    for (int k16 = 0; k16 < BK / 16; ++k16)
                        mma_ss(d, smem_desc_sw128(a, k16 * 32), smem_desc_sw128(b, k16 * 32), idesc, kb > 0 || k16 > 0);
                    mma_commit(smem_u32(&empty_bar[s]));    // the stage is free once these MMAs have read it
                }
                mma_commit(smem_u32(&acc_full[buf]));       // this tile's accumulator is complete
            }
        }
    } else {                                                // ---- epilogue: TMEM lanes by warp % 4
        const int q = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const Tile t = locate(s_start, s_off, E, N, total_m, tile);
            const int buf = local & 1;
            ok = mbar_wait(smem_u32(&acc_full[buf]), (local >> 1) & 1) && ok;
            if (tile + (int)gridDim.x >= tiles) pdl_trigger_late();        // the last tile of this CTA
            fence_after_sync();
            const int r_local = q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tmem_ld32(tacc + ((unsigned)(q * 32) << 16) + buf * BN + c0, r);
                tmem_ld_wait();
                if (r_local >= t.rows || t.n0 + c0 >= N) continue;
                store_chunk(out + (size_t)(t.m0 + r_local) * ldo + t.n0 + c0, r, min(32, N - t.n0 - c0));
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));         // this warp has drained its quarter
        }
    }
    if (!ok) atomicExch(status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tacc, TMEM_COLS);
}

}  // namespace

// A [places, K] (the pairs' rows in the order of their experts), W [E, N, K] contiguous, offsets int32 [E + 1] on the
// device, out [places, N] bfloat16.  status: one int in device memory, set to 1 if a wait inside the kernel gave up.
RB_EXPORT int rb_moe_tc5_gemm(const void* A, int lda, const void* W, const int* offsets, int E, void* out, int ldo, int places,
                              int N, int K, int* status, cudaStream_t st) {
    if (places <= 0 || N <= 0) return 0;
    if (E > MAX_EXPERTS || K % 8 || lda % 8 || ((uintptr_t)A % 16) || ((uintptr_t)W % 16)) return (int)cudaErrorInvalidValue;
    if ((long long)E * N > 0x7fffffffLL) return (int)cudaErrorInvalidValue;
    CUtensorMap ma, mw;
    if (!tma::make_map_bf16(&ma, A, places, K, lda, BM) || !tma::make_map_bf16(&mw, W, E * N, K, K, BN)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)STAGES * (BM + BN) * BK * 2 + 1024;
    static PerDevice configured;
    const int rc = configured.once([&](int) {
        return cudaFuncSetAttribute(moe_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (rc != 0) return rc;
    const long long worst = ((long long)(places + BM - 1) / BM + E) * ((N + BN - 1) / BN);
    const int num_sms = rb_num_sms();
    if (num_sms <= 0) return (int)cudaErrorInvalidDevice;
    dim3 grid((unsigned)(worst < num_sms ? worst : num_sms));
    return rb_launch_pdl(moe_tc5_kernel, grid, dim3(THREADS), smem, st, ma, mw, offsets, E, (bf16*)out, N, K, ldo, status);
}
