// Several residual streams ("hyper-connections"): instead of one stream x a model keeps S streams
// x_1 .. x_S.  A sublayer reads u = sum_s in[s] x_s through its norm, and its output y goes back into
// all streams at once, x_t <- sum_s mix[s][t] x_s + out[t] y.
//
//   tuff_hc_step   one launch between two sublayers: applies the update that the last sublayer left
//                  (its y, mix and out; or copies a fresh stream into all S; or nothing), then reads the
//                  next sublayer's input out of the new streams, u = sum_t in[t] x_t (in = null: the plain
//                  sum), and norms it, h = u * rsqrt(mean(u^2) + eps) * w, in the activation's type.
//                  y is cleared after it was read, so the sublayer that follows can add into it again.
//   tuff_relu2     z <- max(z, 0)^2 in place, the activation of a feed-forward without a gate.
//
// Everything is fp32 but h.  One block per token; a thread's columns (four neighbours at a time where the width
// is a multiple of four) and the order of every sum depend on the width and the alignment alone, so a token's result does not depend on the batch it is in.
#include "common.cuh"

namespace {
constexpr int HC_MAX_S = 8;
constexpr int HC_THREADS = 256;

struct HcParams {
    float* X;              // [S, T, d] the streams
    const float* x_init;   // [T, d] or null: every stream starts as this row
    float* y;              // [T, d] or null: the finished sublayer's output
    const float* mix;      // [S, S] indexed [from][to]
    const float* outw;     // [S]
    const float* inw;      // [S] or null (all ones)
    const float* norm_w;   // [d] or null (h is u itself)
    void* h_out;           // [T, d] or null
    float* u_out;          // [T, d] or null
    int S, T, d;
    float eps;
    int zero_y;
};

// V consecutive columns (1, or 4 where the width and the pointers allow: one 16-byte access each).
template <int V> struct HcVec { float v[V]; };
template <int V> __device__ __forceinline__ HcVec<V> hc_load(const float* p) {
    HcVec<V> r;
    if constexpr (V == 4) { const float4 q = __ldcg(reinterpret_cast<const float4*>(p)); r.v[0] = q.x; r.v[1] = q.y; r.v[2] = q.z; r.v[3] = q.w; }
    else r.v[0] = ld_act(p);
    return r;
}
template <int V> __device__ __forceinline__ void hc_store(float* p, const HcVec<V>& r) {
    if constexpr (V == 4) *reinterpret_cast<float4*>(p) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    else *p = r.v[0];
}

template <typename TH, int S, int V>
__global__ void __launch_bounds__(HC_THREADS)
hc_step_kernel(HcParams p) {
    extern __shared__ __align__(16) float u_row[];           // [d]
    __shared__ float scratch[32];
    __shared__ float sh_mix[HC_MAX_S * HC_MAX_S], sh_out[HC_MAX_S], sh_in[HC_MAX_S];
    const int t = blockIdx.x;
    // the small weights are no kernel's output: they may be read before the predecessor has finished
    if (threadIdx.x < S * S) sh_mix[threadIdx.x] = p.mix ? p.mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        sh_out[threadIdx.x] = p.outw ? p.outw[threadIdx.x] : 0.f;
        sh_in[threadIdx.x] = p.inw ? p.inw[threadIdx.x] : 1.f;
    }
    pdl_wait();
    pdl_launch_dependents();
    __syncthreads();
    const size_t row = (size_t)t * p.d, plane = (size_t)p.T * p.d;
    float ss = 0.f;
    for (int c = threadIdx.x * V; c < p.d; c += HC_THREADS * V) {
        HcVec<V> nx[S];
        if (p.x_init) {
            const HcVec<V> v = hc_load<V>(p.x_init + row + c);
#pragma unroll
            for (int s = 0; s < S; ++s) { nx[s] = v; hc_store<V>(p.X + s * plane + row + c, v); }
        } else {
            HcVec<V> x[S];
#pragma unroll
            for (int s = 0; s < S; ++s) x[s] = hc_load<V>(p.X + s * plane + row + c);
            if (p.y) {
                const HcVec<V> yv = hc_load<V>(p.y + row + c);
#pragma unroll
                for (int to = 0; to < S; ++to) {
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        float a = 0.f;
#pragma unroll
                        for (int s = 0; s < S; ++s) a = fmaf(sh_mix[s * S + to], x[s].v[e], a);
                        nx[to].v[e] = fmaf(sh_out[to], yv.v[e], a);
                    }
                    hc_store<V>(p.X + to * plane + row + c, nx[to]);
                }
                if (p.zero_y) { HcVec<V> z; for (int e = 0; e < V; ++e) z.v[e] = 0.f; hc_store<V>(p.y + row + c, z); }
            } else {
#pragma unroll
                for (int s = 0; s < S; ++s) nx[s] = x[s];
            }
        }
        HcVec<V> u;
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s) a = fmaf(sh_in[s], nx[s].v[e], a);
            u.v[e] = a;
            ss = fmaf(a, a, ss);
        }
        hc_store<V>(u_row + c, u);
        if (p.u_out) hc_store<V>(p.u_out + row + c, u);
    }
    if (!p.h_out) return;
    float r = 1.f;
    if (p.norm_w) r = rsqrtf(block_sum(ss, scratch) / (float)p.d + p.eps);
    TH* h = reinterpret_cast<TH*>(p.h_out) + row;
    for (int c = threadIdx.x * V; c < p.d; c += HC_THREADS * V) {      // each thread re-reads what it wrote itself
#pragma unroll
        for (int e = 0; e < V; ++e)
            h[c + e] = from_f32<TH>(p.norm_w ? u_row[c + e] * r * p.norm_w[c + e] : u_row[c + e]);
    }
}

template <typename T>
__global__ void relu2_kernel(T* z, long long n) {
    pdl_wait();
    pdl_launch_dependents();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        const float v = fmaxf(ld_act(z + i), 0.f);
        z[i] = from_f32<T>(v * v);
    }
}

template <typename TH, int V>
int hc_launch_v(const HcParams& p, cudaStream_t stream) {
    const size_t smem = (size_t)p.d * sizeof(float);
#define HC_GO(S) case S: return launch_pdl(hc_step_kernel<TH, S, V>, dim3(p.T), dim3(HC_THREADS), smem, stream, p)
    switch (p.S) { HC_GO(1); HC_GO(2); HC_GO(3); HC_GO(4); HC_GO(5); HC_GO(6); HC_GO(7); HC_GO(8); }
#undef HC_GO
    return TUFF_E_SIZE;
}
template <typename TH>
int hc_launch(const HcParams& p, cudaStream_t stream) {
    // 16-byte accesses where every row starts on one: the width a multiple of 4 and the bases aligned
    const uintptr_t bases = (uintptr_t)p.X | (uintptr_t)p.x_init | (uintptr_t)p.y | (uintptr_t)p.u_out;
    if (p.d % 4 == 0 && (bases & 15) == 0) return hc_launch_v<TH, 4>(p, stream);
    return hc_launch_v<TH, 1>(p, stream);
}
}  // namespace

// X [S, T, d] fp32.  x_init (else y with mix [S, S] and outw [S], else nothing) says how the streams change
// first; inw [S] (null: ones) and norm_w [d] (null: no norm) say what is read out into h_out (h_dtype) and
// u_out (the unnormed fp32 sum); either may be null.  zero_y: y is cleared once read.
extern "C" int tuff_hc_step(float* X, int S, int T, int d, const float* x_init, float* y, const float* mix,
                            const float* outw, const float* inw, const float* norm_w, float eps, void* h_out,
                            int h_dtype, float* u_out, int zero_y, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (S < 1 || S > HC_MAX_S || d < 1 || d > 12288) return TUFF_E_SIZE;     // a row of u in 48 KB of shared memory
    if (y && (!mix || !outw)) return TUFF_E_SIZE;
    HcParams p{X, x_init, y, mix, outw, inw, norm_w, h_out, u_out, S, T, d, eps, zero_y};
    if (h_dtype == TUFF_F32) return hc_launch<float>(p, stream);
    if (h_dtype == TUFF_BF16) return hc_launch<bf16>(p, stream);
    return TUFF_E_DTYPE;
}

extern "C" int tuff_relu2(void* z, int dtype, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const unsigned blocks = (unsigned)((n + 255) / 256);
    if (dtype == TUFF_F32) return launch_pdl(relu2_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)z, n);
    if (dtype == TUFF_BF16) return launch_pdl(relu2_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)z, n);
    return TUFF_E_DTYPE;
}
