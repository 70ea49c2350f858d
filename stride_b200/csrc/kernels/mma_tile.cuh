// A 64 x 64 output tile of C = A B^T in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulators), for
// the small products that sit between the library products of a layer: the per-head products of latent attention
// and the experts' products, whose rows are scattered or ragged. Four warps, each 32 x 32 of the tile; operands are
// staged in shared memory 64 columns of K at a time (rows padded by 8 elements: the fragment loads of a warp then fall
// into 32 different banks) and read as the instruction's fragments with ldmatrix.
//
//   A: row r of the tile starts at a_rows[r] (nullptr: the row is beyond the end and counts as zeros), K contiguous.
//   B: element (n, k) at B[n * b_ns + k * b_ks]; either stride may be 1.
// Every output element is a sum over k in the order of the instruction, the same for any tile and any batch, so a row's
// result does not depend on what else is computed beside it.
#pragma once

#include "common.cuh"

namespace stride {

constexpr int TM = 64, TN = 64, TK = 64, TPAD = TK + 8;
constexpr int TCH = TK / 8;                 // 16-byte pieces a row and step
constexpr int TPIECES = TM * TCH / 128;     // pieces of A (and of B) a thread and step

struct __align__(16) TileSmem {
    __nv_bfloat16 a[TM][TPAD];
    __nv_bfloat16 b[TN][TPAD];
    const __nv_bfloat16* a_rows[TM];
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Four 8 x 8 matrices of 16-bit numbers from shared memory, one row address a lane: lanes 0-7 name the rows of the first
// matrix, 8-15 of the second, and so on; register k of a lane holds its two elements of matrix k.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(smem_row));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// acc[i][j][.]: the warp's m16 tile i (rows wm * 32 + i * 16 ..) and n8 tile j (columns wn * 32 + j * 8 ..), wm = warp / 2,
// wn = warp % 2. Element e of a fragment: row (lane / 4) + 8 * (e / 2), column 2 * (lane % 4) + (e % 2).
// Call with 128 threads; sm.a_rows must be filled and visible (__syncthreads) before.
__device__ __forceinline__ void mma_tile_64x64(TileSmem& sm, const __nv_bfloat16* __restrict__ B, long long b_ns, long long b_ks, int n0,
                                               int N, int K, float (&acc)[2][4][4]) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;
    // Each thread fetches four 16-byte pieces of A and four of B a step (or 16 single elements of B where n is the
    // contiguous index). The pieces of step k + 1 are requested into registers before the products of step k run,
    // so the latency of global memory is covered by arithmetic.
    uint4 pa[TPIECES], pb[TPIECES];
    __nv_bfloat16 pbs[(TN * TK) / 128];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int x = 0; x < TPIECES; ++x) {
            const int c = tid + x * 128;
            const int r = c / TCH, kc = (c % TCH) * 8;
            const __nv_bfloat16* src = sm.a_rows[r];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (src && k0 + kc < K) {
                src += k0 + kc;
                if (k0 + kc + 8 <= K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                    v = *reinterpret_cast<const uint4*>(src);
                } else {
                    __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
                    for (int y = 0; y < 8; ++y)
                        if (k0 + kc + y < K) e[y] = src[y];
                }
            }
            pa[x] = v;
        }
        if (b_ks == 1) {
#pragma unroll
            for (int x = 0; x < TPIECES; ++x) {
                const int c = tid + x * 128;
                const int n = c / TCH, kc = (c % TCH) * 8;
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (n0 + n < N && k0 + kc < K) {
                    const __nv_bfloat16* src = B + static_cast<long long>(n0 + n) * b_ns + k0 + kc;
                    if (k0 + kc + 8 <= K && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
                        v = *reinterpret_cast<const uint4*>(src);
                    } else {
                        __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&v);
                        for (int y = 0; y < 8; ++y)
                            if (k0 + kc + y < K) e[y] = src[y];
                    }
                }
                pb[x] = v;
            }
        } else {        // n contiguous in memory: neighbouring threads read neighbouring n
#pragma unroll
            for (int x = 0; x < (TN * TK) / 128; ++x) {
                const int c = tid + x * 128;
                const int k = c / TN, n = c % TN;
                pbs[x] = (n0 + n < N && k0 + k < K) ? B[static_cast<long long>(n0 + n) * b_ns + static_cast<long long>(k0 + k) * b_ks]
                                                    : __float2bfloat16_rn(0.f);
            }
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int x = 0; x < TPIECES; ++x) {
            const int c = tid + x * 128;
            *reinterpret_cast<uint4*>(&sm.a[c / TCH][(c % TCH) * 8]) = pa[x];
        }
        if (b_ks == 1) {
#pragma unroll
            for (int x = 0; x < TPIECES; ++x) {
                const int c = tid + x * 128;
                *reinterpret_cast<uint4*>(&sm.b[c / TCH][(c % TCH) * 8]) = pb[x];
            }
        } else {
#pragma unroll
            for (int x = 0; x < (TN * TK) / 128; ++x) {
                const int c = tid + x * 128;
                sm.b[c % TN][c / TN] = pbs[x];
            }
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += TK) {
        stash();
        if (k0 + TK < K) fetch(k0 + TK);
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; kk += 16) {
            uint32_t af[2][4], bf[4][2];
            // A: rows (lane % 16) of the m16 tile, columns kk + 8 * (lane / 16): the four matrices are the fragment's a0..a3
#pragma unroll
            for (int i = 0; i < 2; ++i) ldmatrix_x4(af[i], &sm.a[wm * 32 + i * 16 + (lane & 15)][kk + (lane >> 4) * 8]);
            // B: two n8 tiles a load: matrices (n 0-7, k 0-7), (n 0-7, k 8-15), (n 8-15, k 0-7), (n 8-15, k 8-15)
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                uint32_t r[4];
                ldmatrix_x4(r, &sm.b[wn * 32 + j * 8 + (lane & 7) + ((lane >> 4) << 3)][kk + ((lane >> 3) & 1) * 8]);
                bf[j][0] = r[0];
                bf[j][1] = r[1];
                bf[j + 1][0] = r[2];
                bf[j + 1][1] = r[3];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], af[i], bf[j]);
        }
        __syncthreads();
    }
}

// Row and column (inside the tile) of element e of acc[i][j].
__device__ __forceinline__ int tile_row(int i, int e) { return ((threadIdx.x >> 5) >> 1) * 32 + i * 16 + ((threadIdx.x & 31) >> 2) + 8 * (e >> 1); }
__device__ __forceinline__ int tile_col(int j, int e) { return ((threadIdx.x >> 5) & 1) * 32 + j * 8 + 2 * (threadIdx.x & 3) + (e & 1); }

}  // namespace stride
