// Plain CUDA-core matrix product  C[M,N] (=|+=) A[M,K] * W[N,K]^T  with fp32
// accumulation by FFMA: no tensor cores and no reduced-precision mode, so it is
// the product of the true 32-bit path and the fallback of the bf16 path for
// shapes that the tensor-core kernels refuse.
//
// W is [out, in] as the checkpoints store it, the layout the reference's
// matrix-vector kernels read (src/lfm25_gpu.cu:148-202); `accumulate` adds into
// an fp32 C, which is how the residual stream takes a projection's result
// (the reference's accum=true: src/lfm25_engine.c:380,405,419).
//
// Every element of C is summed over k = 0..K-1 in ascending order by one thread,
// so its value does not depend on M, on which rows share a tile, or on the grid.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

template <typename AT, typename WT, typename CT, bool ACCUM>
__global__ void __launch_bounds__(256)
gemm_plain_kernel(const AT* __restrict__ A, const WT* __restrict__ W, CT* __restrict__ C,
                  int M, int N, int K, long long lda, long long ldw, long long ldc,
                  long long sa, long long sw, long long sc) {
    // blockIdx.z: which product of a batch (one per head, say); the strides between them in elements
    A += (size_t)blockIdx.z * sa; W += (size_t)blockIdx.z * sw; C += (size_t)blockIdx.z * sc;
    __shared__ float As[BK][BM + PAD];
    __shared__ float Ws[BK][BN + PAD];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2;          // 0..63: tile row loaded by this thread
    const int lk = (tid & 3) * 4;     // first of its 4 k values
    const int ty = tid >> 4, tx = tid & 15;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        {
            const int gm = m0 + lr, gn = n0 + lr;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int gk = k0 + lk + j;
                As[lk + j][lr] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
                Ws[lk + j][lr] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            CT* p = C + (size_t)gm * ldc + gn;
            if (ACCUM) *p = from_f32<CT>(to_f32(*p) + acc[i][j]);
            else *p = from_f32<CT>(acc[i][j]);
        }
    }
}
// A batch of products with few rows (bf16): C[m, n] = sum_k A[m, k] W[n, k] for up to HR_ROWS rows m per CTA.
// One warp per output column n: its lanes take pairs of k in turn, every lane keeps one sum per row, and the
// lanes' sums are added by shuffles, so an element's value depends on K alone.  The weights are read once
// per HR_ROWS rows, in whole lines.
constexpr int HR_ROWS = 8, HR_WARPS = 8;
__global__ void __launch_bounds__(HR_WARPS * 32)
head_rows_kernel(const bf16* __restrict__ A, const bf16* __restrict__ W, bf16* __restrict__ C, int M, int N, int K,
                 long long lda, long long ldw, long long ldc, long long sa, long long sw, long long sc) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * HR_WARPS + warp, m0 = blockIdx.z * HR_ROWS;
    A += (size_t)blockIdx.y * sa + (size_t)m0 * lda; W += (size_t)blockIdx.y * sw; C += (size_t)blockIdx.y * sc + (size_t)m0 * ldc;
    pdl_wait();
    pdl_launch_dependents();
    if (n >= N) return;
    const int rows = min(HR_ROWS, M - m0);
    float acc[HR_ROWS];
#pragma unroll
    for (int i = 0; i < HR_ROWS; ++i) acc[i] = 0.f;
    const bf16* wrow = W + (size_t)n * ldw;
    for (int k = 2 * lane; k < K; k += 64) {
        const float2 w = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(wrow + k));
#pragma unroll
        for (int i = 0; i < HR_ROWS; ++i) {
            if (i < rows) {
                const uint32_t raw = ld_act_u32(A + (size_t)i * lda + k);
                const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
                acc[i] = fmaf(a.y, w.y, fmaf(a.x, w.x, acc[i]));
            }
        }
    }
    float mine = 0.f;
#pragma unroll
    for (int i = 0; i < HR_ROWS; ++i) {
        const float v = warp_sum(acc[i]);
        if (lane == i) mine = v;
    }
    if (lane < rows) C[(size_t)lane * ldc + n] = __float2bfloat16_rn(mine);
}
// The same batch with the matrices stored [batch][K][N] (N contiguous), bf16: C[m, n] = sum_k A[m, k] Wt[k, n].
// A thread owns one column n for HC_ROWS rows and a quarter of K (threadIdx.y); neighbouring threads read
// neighbouring columns of a row of Wt, the rows of A come from shared memory as broadcasts.  The four partial
// sums are added in the order of the quarters, so an element's value depends on K alone.
constexpr int HC_COLS = 64, HC_KPARTS = 4, HC_ROWS = 8, HC_MAX_K = 1024;
__global__ void __launch_bounds__(HC_COLS * HC_KPARTS)
head_cols_kernel(const bf16* __restrict__ A, const bf16* __restrict__ Wt, bf16* __restrict__ C, int M, int N, int K,
                 long long lda, long long ldc, long long sa, long long sw, long long sc) {
    __shared__ float a_s[HC_ROWS][HC_MAX_K];
    __shared__ float part[HC_KPARTS][HC_ROWS][HC_COLS];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int n = blockIdx.x * HC_COLS + tx, m0 = blockIdx.z * HC_ROWS;
    const int rows = min(HC_ROWS, M - m0);
    A += (size_t)blockIdx.y * sa + (size_t)m0 * lda; Wt += (size_t)blockIdx.y * sw; C += (size_t)blockIdx.y * sc + (size_t)m0 * ldc;
    pdl_wait();
    pdl_launch_dependents();
    for (int i = ty * HC_COLS + tx; i < HC_ROWS * K; i += HC_COLS * HC_KPARTS) {
        const int r = i / K, k = i % K;
        a_s[r][k] = r < rows ? ld_act(A + (size_t)r * lda + k) : 0.f;
    }
    __syncthreads();
    const int per = (K + HC_KPARTS - 1) / HC_KPARTS;
    const int k0 = ty * per, k1 = min(K, k0 + per);
    float acc[HC_ROWS];
#pragma unroll
    for (int i = 0; i < HC_ROWS; ++i) acc[i] = 0.f;
    if (n < N) {
#pragma unroll 4
        for (int k = k0; k < k1; ++k) {
            const float w = __bfloat162float(Wt[(size_t)k * N + n]);
#pragma unroll
            for (int i = 0; i < HC_ROWS; ++i) acc[i] = fmaf(a_s[i][k], w, acc[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < HC_ROWS; ++i) part[ty][i][tx] = acc[i];
    __syncthreads();
    if (n < N) {
        for (int i = ty; i < rows; i += HC_KPARTS) {
            float v = part[0][i][tx];
#pragma unroll
            for (int q = 1; q < HC_KPARTS; ++q) v += part[q][i][tx];
            C[(size_t)i * ldc + n] = __float2bfloat16_rn(v);
        }
    }
}
}  // namespace

// `batch` products in one launch: product b reads A + b*sa, W + b*sw and writes C + b*sc (strides in elements).
// The heads of a projection that has a matrix of its own per head are such a batch: A [M, heads, K] with
// lda = heads*K and sa = K, and so on.
extern "C" int tuff_gemm_plain_batched(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                                       int M, int N, int K, long long lda, long long ldw, long long ldc,
                                       int batch, long long sa, long long sw, long long sc,
                                       int accumulate, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || batch > 65535) return TUFF_E_SIZE;
    dim3 grid(ceil_div(N, BN), ceil_div(M, BM), batch);
#define GO(AT, WT, CT, ACC) gemm_plain_kernel<AT, WT, CT, ACC><<<grid, 256, 0, stream>>>( \
        (const AT*)A, (const WT*)W, (CT*)C, M, N, K, lda, ldw, ldc, sa, sw, sc)
    if (accumulate && c_dtype != TUFF_F32) return TUFF_E_DTYPE;
    if (a_dtype == TUFF_F32 && w_dtype == TUFF_F32 && c_dtype == TUFF_F32) {
        if (accumulate) GO(float, float, float, true); else GO(float, float, float, false);
    } else if (a_dtype == TUFF_BF16 && w_dtype == TUFF_BF16 && c_dtype == TUFF_BF16) {
        GO(bf16, bf16, bf16, false);
    } else if (a_dtype == TUFF_BF16 && w_dtype == TUFF_BF16 && c_dtype == TUFF_F32) {
        if (accumulate) GO(bf16, bf16, float, true); else GO(bf16, bf16, float, false);
    } else if (a_dtype == TUFF_F32 && w_dtype == TUFF_BF16 && c_dtype == TUFF_F32) {
        if (accumulate) GO(float, bf16, float, true); else GO(float, bf16, float, false);
    } else {
        return TUFF_E_DTYPE;
    }
#undef GO
    return launch_status();
}

extern "C" int tuff_gemm_plain(const void* A, int a_dtype, const void* W, int w_dtype, void* C, int c_dtype,
                               int M, int N, int K, long long lda, long long ldw, long long ldc,
                               int accumulate, cudaStream_t stream) {
    return tuff_gemm_plain_batched(A, a_dtype, W, w_dtype, C, c_dtype, M, N, K, lda, ldw, ldc, 1, 0, 0, 0, accumulate, stream);
}

// The same batch for few rows (M small against N), bf16 throughout: one warp per output column.  K and all
// strides even, the pointers 4-byte aligned; else TUFF_E_ALIGN and the caller takes the general kernel.
extern "C" int tuff_head_rows(const void* A, const void* W, void* C, int M, int N, int K, long long lda, long long ldw,
                              long long ldc, int batch, long long sa, long long sw, long long sc, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || batch > 65535 || ceil_div(M, HR_ROWS) > 65535) return TUFF_E_SIZE;
    if ((K | lda | ldw | sa | sw) & 1) return TUFF_E_ALIGN;
    if (((uintptr_t)A | (uintptr_t)W) & 3) return TUFF_E_ALIGN;
    return launch_pdl(head_rows_kernel, dim3(ceil_div(N, HR_WARPS), batch, ceil_div(M, HR_ROWS)), dim3(HR_WARPS * 32), 0, stream,
                      (const bf16*)A, (const bf16*)W, (bf16*)C, M, N, K, lda, ldw, ldc, sa, sw, sc);
}

// The same batch with the matrices given transposed, Wt [batch][K][N] contiguous (product b reads Wt + b*sw), bf16
// throughout, K up to 1,024: a thread per output column.  Larger K: TUFF_E_SIZE, and the caller takes another kernel.
extern "C" int tuff_head_cols(const void* A, const void* Wt, void* C, int M, int N, int K, long long lda, long long ldc,
                              int batch, long long sa, long long sw, long long sc, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || batch <= 0) return 0;
    if (K <= 0 || K > HC_MAX_K || batch > 65535 || ceil_div(M, HC_ROWS) > 65535) return TUFF_E_SIZE;
    return launch_pdl(head_cols_kernel, dim3(ceil_div(N, HC_COLS), batch, ceil_div(M, HC_ROWS)), dim3(HC_COLS, HC_KPARTS), 0, stream,
                      (const bf16*)A, (const bf16*)Wt, (bf16*)C, M, N, K, lda, ldc, sa, sw, sc);
}
