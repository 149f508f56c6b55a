// Attention over a latent cache: per token the cache holds one small vector c (the "latent", RMS-normed)
// and one rotated key part kr that all heads share; a head's keys and values are linear images of c,
// k_h = [U_h c | kr], v_h = V_h c.  Instead of expanding every cached token, the query is carried into
// the latent space, q~_h = [U_h^T q_h(plain) | q_h(rotated)], so that q_h . k_h = q~_h . [c | kr]: attention
// then runs with one shared key/value head whose keys are the cached rows [c | kr] and whose values are the
// first `rank` elements of the same rows, and V_h is applied to the weighted sum of latents afterwards.
//
//   tuff_latent_prepare   per token: c = rmsnorm(first `rank` outputs of the down-projection) * w and the
//                         rotated kr, both stored in the request's page row [c | kr]; the rotated parts of
//                         the query heads, stored behind where the absorbed plain parts go ([rank .. rank+rd)
//                         of every head of the latent query).
//
// The rotation pairs neighbouring elements (2i, 2i+1), i < rot_dims/2, turning them by pos * inv_freq[i];
// elements from rot_dims on pass unchanged.  Norm, angles and rotation are fp32.
#include "common.cuh"
#include "index.cuh"

namespace {
constexpr int LP_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(LP_THREADS)
latent_prepare_kernel(const T* __restrict__ qd, long long qd_stride, T* __restrict__ ql, const float* __restrict__ c_norm_w,
                      const float* __restrict__ inv_freq, const int* __restrict__ positions,
                      const int* __restrict__ row_of_token, const int* __restrict__ block_table, int max_blocks,
                      T* __restrict__ k_pages, int H, int dim, int rd, int rank, int rot_dims, int page_size, float eps,
                      int write_kv, Bounds bounds) {
    __shared__ float scratch[32];
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const int pos = ld_act(positions + t);
    const int r = ld_act(row_of_token + t);
    const T* row = qd + (size_t)t * qd_stride;
    const int hq = dim + rd, hl = rank + rd;            // a query head as projected, and in the latent space
    const T* down = row + (size_t)H * hq;               // [c (rank) | kr (rd)]
    const int half = rot_dims >> 1;

    // the rotated parts of the query heads
    T* qrow = ql + (size_t)t * H * hl;
    for (int i = threadIdx.x; i < H * (rd >> 1); i += LP_THREADS) {
        const int h = i / (rd >> 1), j = i % (rd >> 1);
        const float u = ld_act(row + (size_t)h * hq + dim + 2 * j), v = ld_act(row + (size_t)h * hq + dim + 2 * j + 1);
        float sn = 0.f, cs = 1.f;
        if (j < half) sincosf((float)pos * inv_freq[j], &sn, &cs);
        qrow[(size_t)h * hl + rank + 2 * j] = from_f32<T>(u * cs - v * sn);
        qrow[(size_t)h * hl + rank + 2 * j + 1] = from_f32<T>(v * cs + u * sn);
    }
    if (!write_kv) return;

    long long page = -1;
    if (check_row(bounds, r) && check_entry(bounds, pos, page_size, max_blocks)) {
        page = ld_act(block_table + (size_t)r * max_blocks + page_entry(pos, page_size));
        if (!check_page(bounds, page)) page = -1;
    }
    if (TUFF_CHECKED && page < 0) return;
    T* dst = k_pages + page_elem(page, 0, page_offset(pos, page_size), 1, page_size, hl);

    float ss = 0.f;
    for (int e = threadIdx.x; e < rank; e += LP_THREADS) { const float v = ld_act(down + e); ss = fmaf(v, v, ss); }
    const float inv = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int e = threadIdx.x; e < rank; e += LP_THREADS) dst[e] = from_f32<T>(ld_act(down + e) * inv * c_norm_w[e]);
    for (int j = threadIdx.x; j < (rd >> 1); j += LP_THREADS) {
        const float u = ld_act(down + rank + 2 * j), v = ld_act(down + rank + 2 * j + 1);
        float sn = 0.f, cs = 1.f;
        if (j < half) sincosf((float)pos * inv_freq[j], &sn, &cs);
        dst[rank + 2 * j] = from_f32<T>(u * cs - v * sn);
        dst[rank + 2 * j + 1] = from_f32<T>(v * cs + u * sn);
    }
}
}  // namespace

// qd [n, >= H*(dim+rd) + rank + rd] (row stride qd_stride): the stacked projection [q heads | c | kr].
// ql [n, H, rank + rd]: receives the rotated query parts in columns [rank, rank + rd) of every head.
// k_pages [pages, 1, page_size, rank + rd]; write_kv = 0 leaves the pages alone.
extern "C" int tuff_latent_prepare(const void* qd, long long qd_stride, void* ql, int dtype, const float* c_norm_w,
                                   const float* inv_freq, const int* positions, const int* row_of_token,
                                   const int* block_table, int max_blocks, void* k_pages, int n_tokens, int H, int dim,
                                   int rd, int rank, int rot_dims, int page_size, float eps, int write_kv,
                                   long long table_rows, long long n_pages, int* status, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || dim < 1 || rank < 1 || rd < 0 || (rd & 1) || rot_dims < 0 || rot_dims > rd || (rot_dims & 1)) return TUFF_E_SIZE;
    if (write_kv && page_size < 1) return TUFF_E_SIZE;
#define LP_GO(T) return launch_pdl(latent_prepare_kernel<T>, dim3(n_tokens), dim3(LP_THREADS), 0, stream, \
        (const T*)qd, qd_stride, (T*)ql, c_norm_w, inv_freq, positions, row_of_token, block_table, max_blocks, \
        (T*)k_pages, H, dim, rd, rank, rot_dims, page_size, eps, write_kv, Bounds{table_rows, n_pages, status})
    if (dtype == TUFF_F32) LP_GO(float);
    if (dtype == TUFF_BF16) LP_GO(bf16);
#undef LP_GO
    return TUFF_E_DTYPE;
}
