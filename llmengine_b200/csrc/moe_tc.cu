// The grouped product of a mixture of experts on the tensor cores (bfloat16 operands, 32-bit sums): one product per
// expert over the (token, choice) pairs that were routed to it, rows gathered by token on the way in and scattered by
// pair on the way out where asked, silu(gate) * up in the epilogue of the gate|up product.
//
// A block owns a tile of BM pairs of ONE expert x BN output columns and walks K in steps of 32 through a cp.async
// pipeline of two or three stages; its four warps share the tile by columns (mma.sync m16n8k16, fragments by ldmatrix).
// Two shapes: 64 x 64 where experts get many rows (prompts; tiles of 128 rows on eight warps were no faster, 406 against
// 372 us for 2,048 tokens on 4 of 32 experts of 1,024: an expert's last tile is the emptier the larger the tiles are),
// 16 x 128 where they get a few (decode steps: every weight tile is then read by exactly one block, which is all a
// weight-streaming product can ask for).  The row tiles of all experts
// are numbered one after the other and a block finds its expert from the offsets; a launch has as many row tiles as
// any routing can need, and blocks beyond the step's own count leave at once.  A row's sums never depend on which
// other rows share its tile.
#include "common.cuh"
#include "kernel_args.h"

LLME_API const char* llme_last_error() { return llme_error_buffer(); }

namespace {

typedef __nv_bfloat16 bf16;
constexpr int BK = 32, LDS = BK + 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;                     // 0: the 16 bytes are zero-filled and nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* smem) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* d, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int E, int BM, int tile, int* expert, int* first, int* rows) {
    int seen = 0;
    for (int e = 0; e < E; ++e) {
        const int lo = offsets[e], n = offsets[e + 1] - lo;
        const int tiles = (n + BM - 1) / BM;
        if (tile < seen + tiles) {
            const int at = (tile - seen) * BM;
            *expert = e;
            *first = lo + at;
            *rows = n - at < BM ? n - at : BM;
            return true;
        }
        seen += tiles;
    }
    return false;
}

template <typename O> __device__ __forceinline__ void store2(O* p, float a, float b, bool two);
template <> __device__ __forceinline__ void store2<float>(float* p, float a, float b, bool two) {
    p[0] = a;
    if (two) p[1] = b;
}
template <> __device__ __forceinline__ void store2<bf16>(bf16* p, float a, float b, bool two) {
    p[0] = __float2bfloat16_rn(a);
    if (two) p[1] = __float2bfloat16_rn(b);
}

// BM x BN tile on WM x WNW warps, STAGES stages; ACT: the weight rows of a column are its gate row and, n_out further on, its up row.
template <int BM, int BN, int WM, int WNW, int STAGES, bool ACT, typename O>
__global__ void __launch_bounds__(32 * WM * WNW) grouped_tc_kernel(LlmeGroupedArgs a) {
    constexpr int THREADS = 32 * WM * WNW, MT = BM / WM / 16, WN = BN / WNW, NT = WN / 8, HALVES = ACT ? 2 : 1;
    constexpr int A_STAGE = BM * LDS, B_STAGE = HALVES * BN * LDS;
    static_assert(MT >= 1 && NT >= 2 && NT % 2 == 0, "warp tiles are whole 16 x 16 pieces");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* As = reinterpret_cast<bf16*>(smem_raw);                      // [STAGES][BM][LDS]
    bf16* Bs = As + STAGES * A_STAGE;                                  // [STAGES][HALVES][BN][LDS]
    __shared__ int s_tile[3];
    __shared__ int s_src[BM], s_dst[BM];
    pdl_launch_dependents();
    pdl_wait();                                           // the offsets and the order come from the kernel before
    if (threadIdx.x == 0) {
        int e = -1, first = 0, rows = 0;
        if (!find_tile(a.offsets, a.num_experts, BM, blockIdx.y, &e, &first, &rows)) e = -1;
        s_tile[0] = e; s_tile[1] = first; s_tile[2] = rows;
    }
    __syncthreads();
    const int e = s_tile[0], first = s_tile[1], rows = s_tile[2];
    if (e < 0) return;
    for (int r = threadIdx.x; r < BM; r += THREADS) {
        const int pair = r < rows ? a.order[first + r] : -1;
        s_src[r] = r < rows ? (a.gather ? pair / a.top_k : first + r) : -1;
        s_dst[r] = r < rows ? (a.scatter ? pair : first + r) : -1;
    }
    __syncthreads();
    const int n_out = ACT ? a.n / 2 : a.n;
    const int col0 = blockIdx.x * BN;
    const bf16* x = (const bf16*)a.x;
    const bf16* w = (const bf16*)a.w + (size_t)e * a.w_expert;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int wm = warp / WNW, wn = warp % WNW;
    const int steps = (a.k + BK - 1) / BK;

    auto load_stage = [&](int stage, int step) {
        if (step < steps) {
            const int k0 = step * BK;
            for (int i = threadIdx.x; i < BM * (BK / 8); i += THREADS) {
                const int r = i / (BK / 8), c = (i % (BK / 8)) * 8;
                const int src = s_src[r];
                const bool ok = src >= 0 && k0 + c < a.k;
                cp_async16(As + stage * A_STAGE + r * LDS + c, ok ? x + (size_t)src * a.ldx + k0 + c : x, ok);
            }
            for (int i = threadIdx.x; i < HALVES * BN * (BK / 8); i += THREADS) {
                const int half = i / (BN * (BK / 8)), r = (i / (BK / 8)) % BN, c = (i % (BK / 8)) * 8;
                const bool ok = col0 + r < n_out && k0 + c < a.k;
                cp_async16(Bs + stage * B_STAGE + (half * BN + r) * LDS + c, ok ? w + (size_t)(half * n_out + col0 + r) * a.ldw + k0 + c : w, ok);
            }
        }
        cp_async_commit();                                // one group a step, also an empty one: the count below relies on it
    };

    float acc[HALVES][MT][NT][4];
#pragma unroll
    for (int h = 0; h < HALVES; ++h)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[h][m][n][i] = 0.0f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) load_stage(s, s);
    for (int s = 0; s < steps; ++s) {
        cp_async_wait<STAGES - 2>();                      // the loads of step s have landed
        __syncthreads();                                  // ... for every thread, and step s - 1 has been read by all
        load_stage((s + STAGES - 1) % STAGES, s + STAGES - 1);
        const bf16* At = As + (s % STAGES) * A_STAGE + wm * (BM / WM) * LDS;
        const bf16* Bt = Bs + (s % STAGES) * B_STAGE;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            unsigned af[MT][4];
#pragma unroll
            for (int m = 0; m < MT; ++m)
                ldmatrix_x4(af[m][0], af[m][1], af[m][2], af[m][3], At + (m * 16 + (lane & 15)) * LDS + kk + (lane >> 4) * 8);
#pragma unroll
            for (int h = 0; h < HALVES; ++h)
#pragma unroll
                for (int n = 0; n < NT; n += 2) {
                    unsigned b0, b1, b2, b3;              // (n-tile n: k 0-7, k 8-15), (n-tile n + 1: k 0-7, k 8-15)
                    ldmatrix_x4(b0, b1, b2, b3, Bt + (h * BN + wn * WN + n * 8 + (lane & 7) + (lane >> 4) * 8) * LDS + kk + ((lane >> 3) & 1) * 8);
#pragma unroll
                    for (int m = 0; m < MT; ++m) {
                        mma_bf16(acc[h][m][n], af[m], b0, b1);
                        mma_bf16(acc[h][m][n + 1], af[m], b2, b3);
                    }
                }
        }
    }

    O* out = (O*)a.out;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int half_rows = 0; half_rows < 2; ++half_rows) {
            const int r = wm * (BM / WM) + m * 16 + (lane >> 2) + half_rows * 8;
            const int dst = s_dst[r];
            if (dst < 0) continue;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int col = col0 + wn * WN + n * 8 + (lane & 3) * 2;
                if (col >= n_out) continue;
                float v0 = acc[0][m][n][half_rows * 2], v1 = acc[0][m][n][half_rows * 2 + 1];
                if (ACT) {
                    // gate and up pass through bfloat16 first, as they do when the activation is a kernel of its own
                    const float g0 = __bfloat162float(__float2bfloat16_rn(v0)), g1 = __bfloat162float(__float2bfloat16_rn(v1));
                    const float u0 = __bfloat162float(__float2bfloat16_rn(acc[HALVES - 1][m][n][half_rows * 2]));
                    const float u1 = __bfloat162float(__float2bfloat16_rn(acc[HALVES - 1][m][n][half_rows * 2 + 1]));
                    v0 = silu_mul_bf16(g0, u0);
                    v1 = silu_mul_bf16(g1, u1);
                }
                store2<O>(out + (size_t)dst * a.ldo + col, v0, v1, col + 1 < n_out);
            }
        }
}

template <int BM, int BN, int WM, int WNW, int STAGES, bool ACT, typename O>
int launch(const LlmeGroupedArgs& a, cudaStream_t s) {
    constexpr int SMEM = STAGES * (BM + (ACT ? 2 : 1) * BN) * LDS * (int)sizeof(bf16);
    const int n_out = ACT ? a.n / 2 : a.n;
    const int most = a.num_experts < a.pairs ? a.num_experts : a.pairs;
    int tiles = (a.pairs + BM - 1) / BM + most;           // every expert may add one tile that is not full
    if (tiles > a.pairs) tiles = a.pairs;
    if (tiles > 65535) {
        snprintf(llme_error_buffer(), 512, "grouped_linear_tc: %d row tiles exceed a launch", tiles);
        return -1;
    }
    auto kernel = grouped_tc_kernel<BM, BN, WM, WNW, STAGES, ACT, O>;
    static bool configured = false;
    if (!configured) {
        if (SMEM > 48 * 1024 && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
            snprintf(llme_error_buffer(), 512, "grouped_linear_tc: %d bytes of shared memory are not available", SMEM);
            return -1;
        }
        configured = true;
    }
    llme_launch(kernel, dim3((n_out + BN - 1) / BN, tiles), dim3(32 * WM * WNW), (size_t)SMEM, s, a);
    LLME_LAUNCH_STATUS();
}

template <bool ACT, typename O>
int dispatch(const LlmeGroupedArgs& a, cudaStream_t s) {
    // few rows per expert: tiles of 16 rows, so that little of a tile is padding and every weight is read once
    if ((long long)a.pairs < 32LL * a.num_experts) return launch<16, 128, 1, 4, 4, ACT, O>(a, s);     // three steps of weights in flight per block
    return launch<64, 64, 1, 4, 3, ACT, O>(a, s);
}

}  // namespace

LLME_API int llme_grouped_linear_tc(const LlmeGroupedArgs* args, int x_dtype, int w_dtype, int out_dtype, cudaStream_t stream) {
    const LlmeGroupedArgs& a = *args;
    if (a.pairs <= 0 || a.n <= 0) return 0;
    if (!a.x || !a.w || !a.out || !a.offsets || !a.order) LLME_REFUSE("grouped_linear_tc: null pointer");
    if (x_dtype != LLME_BF16 || w_dtype != LLME_BF16) LLME_REFUSE("grouped_linear_tc: bfloat16 operands only");
    if (a.num_experts <= 0 || a.top_k <= 0 || a.k <= 0 || (a.act && a.n % 2)) LLME_REFUSE("grouped_linear_tc: bad size");
    if (a.k % 8 || a.ldx % 8 || a.ldw % 8 || a.w_expert % 8 || (((uintptr_t)a.x | (uintptr_t)a.w) & 15))
        LLME_REFUSE("grouped_linear_tc: rows must be whole 16-byte pieces");
    if (a.act && out_dtype == LLME_BF16) return dispatch<true, bf16>(a, stream);
    if (a.act && out_dtype == LLME_F32) return dispatch<true, float>(a, stream);
    if (!a.act && out_dtype == LLME_BF16) return dispatch<false, bf16>(a, stream);
    if (!a.act && out_dtype == LLME_F32) return dispatch<false, float>(a, stream);
    LLME_REFUSE("grouped_linear_tc: unsupported output dtype %d", out_dtype);
}
