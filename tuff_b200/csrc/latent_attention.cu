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
                      int write_kv, Bounds bounds, int q_in_place) {
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

    // the rotated parts of the query heads: into the latent query, or back where they came from (each pair is read
    // and written by the same thread)
    T* qrow = q_in_place ? const_cast<T*>(row) + dim : ql + (size_t)t * H * hl + rank;
    const int q_head = q_in_place ? hq : hl;
    for (int i = threadIdx.x; i < H * (rd >> 1); i += LP_THREADS) {
        const int h = i / (rd >> 1), j = i % (rd >> 1);
        const float u = ld_act(row + (size_t)h * hq + dim + 2 * j), v = ld_act(row + (size_t)h * hq + dim + 2 * j + 1);
        float sn = 0.f, cs = 1.f;
        if (j < half) sincosf((float)pos * inv_freq[j], &sn, &cs);
        qrow[(size_t)h * q_head + 2 * j] = from_f32<T>(u * cs - v * sn);
        qrow[(size_t)h * q_head + 2 * j + 1] = from_f32<T>(v * cs + u * sn);
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
// ---- expanding cached latents into keys and values per head, for portions of prompts ----------------------------
// A prompt portion has as many queries as keys, so there it is cheaper to expand the cached rows once,
// k_h = [U_h c | kr] and v_h = V_h c, and to run ordinary attention with heads of dim + rd, than to carry every
// query into the latent space.  The rows of the requests in question are laid out in scratch pages of
// SCRATCH_PAGE tokens: page p holds positions pos0 .. pos0 + n - 1 of row `row` (meta[p] = {row, pos0, n, 0}).
constexpr int SCRATCH_PAGE = 64;

// c_out [pages * SCRATCH_PAGE, rank]: the latents of the scratch pages' tokens (zeros past a row's end).
__global__ void __launch_bounds__(128)
latent_gather_kernel(const bf16* __restrict__ k_pages, const int* __restrict__ block_table, int max_blocks,
                     const int* __restrict__ meta, bf16* __restrict__ c_out, int rank, int hl, int page_size, Bounds bounds) {
    const int p = blockIdx.x / SCRATCH_PAGE, j = blockIdx.x % SCRATCH_PAGE;
    pdl_wait();
    pdl_launch_dependents();
    const int row = ld_act(meta + 4 * p), pos = ld_act(meta + 4 * p + 1) + j, n = ld_act(meta + 4 * p + 2);
    uint4* dst = reinterpret_cast<uint4*>(c_out + (size_t)blockIdx.x * rank);
    const uint4* src = nullptr;
    if (j < n && check_row(bounds, row) && check_entry(bounds, pos, page_size, max_blocks)) {
        const long long page = ld_act(block_table + (size_t)row * max_blocks + page_entry(pos, page_size));
        if (check_page(bounds, page))
            src = reinterpret_cast<const uint4*>(k_pages + page_elem(page, 0, page_offset(pos, page_size), 1, page_size, hl));
    }
    for (int e = threadIdx.x; e < rank / 8; e += blockDim.x) dst[e] = src ? ld_act_u4(src + e) : make_uint4(0u, 0u, 0u, 0u);
}

// kv [pages * SCRATCH_PAGE, H*dim + H*vd]: the expanded plain key parts and values of the scratch tokens.  Stores
// k_out [pages, H, SCRATCH_PAGE, dim + rd] = [plain part | kr from the cache] and v_out [pages, H, SCRATCH_PAGE, vd].
__global__ void __launch_bounds__(128)
latent_expand_store_kernel(const bf16* __restrict__ kv, const bf16* __restrict__ k_pages, const int* __restrict__ block_table,
                           int max_blocks, const int* __restrict__ meta, bf16* __restrict__ k_out, bf16* __restrict__ v_out,
                           int H, int dim, int rd, int vd, int rank, int page_size, Bounds bounds) {
    const int p = blockIdx.x / SCRATCH_PAGE, j = blockIdx.x % SCRATCH_PAGE;
    pdl_wait();
    pdl_launch_dependents();
    const int row = ld_act(meta + 4 * p), pos = ld_act(meta + 4 * p + 1) + j, n = ld_act(meta + 4 * p + 2);
    const int hl = rank + rd, hq = dim + rd;
    const uint4* kr = nullptr;
    if (j < n && check_row(bounds, row) && check_entry(bounds, pos, page_size, max_blocks)) {
        const long long page = ld_act(block_table + (size_t)row * max_blocks + page_entry(pos, page_size));
        if (check_page(bounds, page))
            kr = reinterpret_cast<const uint4*>(k_pages + page_elem(page, 0, page_offset(pos, page_size), 1, page_size, hl) + rank);
    }
    const bf16* src = kv + (size_t)blockIdx.x * ((size_t)H * (dim + vd));
    const int kq = hq / 8, dq = dim / 8, vq = vd / 8;
    for (int i = threadIdx.x; i < H * kq; i += blockDim.x) {
        const int h = i / kq, e = i % kq;
        uint4 v;
        if (e < dq) v = ld_act_u4(reinterpret_cast<const uint4*>(src + (size_t)h * dim) + e);
        else v = kr ? ld_act_u4(kr + (e - dq)) : make_uint4(0u, 0u, 0u, 0u);
        reinterpret_cast<uint4*>(k_out + page_elem(p, h, j, H, SCRATCH_PAGE, hq))[e] = v;
    }
    const bf16* vsrc = src + (size_t)H * dim;
    for (int i = threadIdx.x; i < H * vq; i += blockDim.x) {
        const int h = i / vq, e = i % vq;
        reinterpret_cast<uint4*>(v_out + page_elem(p, h, j, H, SCRATCH_PAGE, vd))[e] =
            ld_act_u4(reinterpret_cast<const uint4*>(vsrc + (size_t)h * vd) + e);
    }
}
}  // namespace

extern "C" int tuff_latent_scratch_page() { return SCRATCH_PAGE; }

// Latents of `n_scratch_pages` scratch pages (see above) into c_out; bf16; rank, rank + rd multiples of 8.
extern "C" int tuff_latent_gather(const void* k_pages, const int* block_table, int max_blocks, const int* meta,
                                  void* c_out, int n_scratch_pages, int rank, int rd, int page_size, long long table_rows,
                                  long long n_pages, int* status, cudaStream_t stream) {
    if (n_scratch_pages <= 0) return 0;
    if (rank < 8 || (rank % 8) || rd < 0 || (rd % 8) || page_size < 1) return TUFF_E_SIZE;
    if (((uintptr_t)k_pages & 15) || ((uintptr_t)c_out & 15)) return TUFF_E_ALIGN;
    return launch_pdl(latent_gather_kernel, dim3(n_scratch_pages * SCRATCH_PAGE), dim3(128), 0, stream,
                      (const bf16*)k_pages, block_table, max_blocks, meta, (bf16*)c_out, rank, rank + rd, page_size,
                      Bounds{table_rows, n_pages, status});
}

// Expanded keys and values of the scratch pages into k_out and v_out; bf16; dim, rd, vd, rank multiples of 8.
extern "C" int tuff_latent_expand_store(const void* kv, const void* k_pages, const int* block_table, int max_blocks,
                                        const int* meta, void* k_out, void* v_out, int n_scratch_pages, int H, int dim,
                                        int rd, int vd, int rank, int page_size, long long table_rows, long long n_pages,
                                        int* status, cudaStream_t stream) {
    if (n_scratch_pages <= 0) return 0;
    if (H < 1 || dim < 8 || (dim % 8) || rd < 0 || (rd % 8) || vd < 8 || (vd % 8) || (rank % 8) || page_size < 1) return TUFF_E_SIZE;
    if (((uintptr_t)kv & 15) || ((uintptr_t)k_pages & 15) || ((uintptr_t)k_out & 15) || ((uintptr_t)v_out & 15)) return TUFF_E_ALIGN;
    return launch_pdl(latent_expand_store_kernel, dim3(n_scratch_pages * SCRATCH_PAGE), dim3(128), 0, stream,
                      (const bf16*)kv, (const bf16*)k_pages, block_table, max_blocks, meta, (bf16*)k_out, (bf16*)v_out,
                      H, dim, rd, vd, rank, page_size, Bounds{table_rows, n_pages, status});
}

// qd [n, >= H*(dim+rd) + rank + rd] (row stride qd_stride): the stacked projection [q heads | c | kr].
// ql [n, H, rank + rd]: receives the rotated query parts in columns [rank, rank + rd) of every head; with
// q_in_place they go back into qd instead (columns [dim, dim + rd) of every head) and ql is not touched.
// k_pages [pages, 1, page_size, rank + rd]; write_kv = 0 leaves the pages alone.
extern "C" int tuff_latent_prepare(const void* qd, long long qd_stride, void* ql, int dtype, const float* c_norm_w,
                                   const float* inv_freq, const int* positions, const int* row_of_token,
                                   const int* block_table, int max_blocks, void* k_pages, int n_tokens, int H, int dim,
                                   int rd, int rank, int rot_dims, int page_size, float eps, int write_kv,
                                   long long table_rows, long long n_pages, int* status, int q_in_place,
                                   cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (H < 1 || dim < 1 || rank < 1 || rd < 0 || (rd & 1) || rot_dims < 0 || rot_dims > rd || (rot_dims & 1)) return TUFF_E_SIZE;
    if (write_kv && page_size < 1) return TUFF_E_SIZE;
#define LP_GO(T) return launch_pdl(latent_prepare_kernel<T>, dim3(n_tokens), dim3(LP_THREADS), 0, stream, \
        (const T*)qd, qd_stride, (T*)ql, c_norm_w, inv_freq, positions, row_of_token, block_table, max_blocks, \
        (T*)k_pages, H, dim, rd, rank, rot_dims, page_size, eps, write_kv, Bounds{table_rows, n_pages, status}, q_in_place)
    if (dtype == TUFF_F32) LP_GO(float);
    if (dtype == TUFF_BF16) LP_GO(bf16);
#undef LP_GO
    return TUFF_E_DTYPE;
}
