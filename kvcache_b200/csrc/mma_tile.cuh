// One output tile of a bfloat16 matrix product on the tensor cores, for kernels whose rows or weights are picked per
// block (a product per head, a product per expert): acc[BM x 64] = A[BM x K] . W[64 x K]^T with mma.sync m16n8k16,
// float32 accumulators, operands brought by cp.async into a ring of stages of rows padded by 16 bytes: tiles of 64 rows
// take 32 of K at a time in two stages, tiles of 16 rows - steps of few rows, which stream their weights once and are
// bound by how many bytes a block keeps in flight - 64 of K in four stages.
//
// A block is 4 warps; warp w owns columns 16 w .. 16 w + 15 of the tile for all MT = BM / 16 row tiles.  `a_row(r)`
// gives the global address of row r's K elements or nullptr (the row is then zero); W rows n >= n_valid are zero.
// K must be a multiple of 8 (16-byte chunks); K is walked in the same order whatever the tile holds, so a row's
// result does not depend on the rows beside it.  `store(row, col, v0, v1)` receives columns col and col + 1.
#pragma once
#include "common.cuh"

namespace mt {

constexpr int BN = 64, THREADS = 128;
template <int MT> struct Shape {
    static constexpr int BK = MT == 1 ? 64 : 32, STAGES = MT == 1 ? 4 : 2, STRIDE = BK + 8;
};

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int MT> struct Smem {
    bf16 a[Shape<MT>::STAGES][16 * MT][Shape<MT>::STRIDE];
    bf16 w[Shape<MT>::STAGES][BN][Shape<MT>::STRIDE];
};

template <int MT, typename ARow, typename Store>
__device__ __forceinline__ void tile_product(Smem<MT>& sm, ARow a_row, const bf16* __restrict__ w, int n_valid, int K, Store store) {
    constexpr int BM = 16 * MT, BK = Shape<MT>::BK, STAGES = Shape<MT>::STAGES, CH = BK / 8;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float acc[MT][2][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f;

    // One group per step of K, also beyond the last step (an empty group), so that "all but the newest STAGES - 2 groups
    // have landed" always means "this step's stage is there".
    auto load = [&](int step, int steps) {
        if (step < steps) {
            const int k0 = step * BK, stage = step % STAGES;
            for (int e = tid; e < BM * CH; e += THREADS) {
                const int r = e / CH, c = (e % CH) * 8;
                const bf16* src = a_row(r);
                const bool valid = src != nullptr && k0 + c < K;
                cp_async16(&sm.a[stage][r][c], valid ? src + k0 + c : w, valid);
            }
            for (int e = tid; e < BN * CH; e += THREADS) {
                const int r = e / CH, c = (e % CH) * 8;
                const bool valid = r < n_valid && k0 + c < K;
                cp_async16(&sm.w[stage][r][c], valid ? w + (size_t)r * K + k0 + c : w, valid);
            }
        }
        cp_async_commit();
    };

    const int steps = (K + BK - 1) / BK;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) load(s, steps);
    for (int s = 0; s < steps; ++s) {
        const int stage = s % STAGES;
        cp_async_wait<STAGES - 2>();
        __syncthreads();                    // step s has landed for every thread, and everyone is done with step s - 1's stage
        load(s + STAGES - 1, steps);        // ... which this refills
#pragma unroll
        for (int ks = 0; ks < BK / 16; ++ks) {
            uint32_t b[4];
            ldmatrix_x4(b[0], b[1], b[2], b[3], &sm.w[stage][warp * 16 + (lane & 7) + (lane >> 4) * 8][ks * 16 + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int i = 0; i < MT; ++i) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], &sm.a[stage][i * 16 + (lane & 15)][ks * 16 + (lane >> 4) * 8]);
                mma_bf16(acc[i][0], a, b[0], b[1]);
                mma_bf16(acc[i][1], a, b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int col = warp * 16 + j * 8 + 2 * t4;
            store(i * 16 + g, col, acc[i][j][0], acc[i][j][1]);
            store(i * 16 + g + 8, col, acc[i][j][2], acc[i][j][3]);
        }
}

}  // namespace mt
