// diopiMm / diopiAddmm / diopiBmm / diopiBaddbmm / diopiMatmul / diopiLinear.
//
// Kernel choice per call:
//   * bf16 / fp16 operands with TMA-compatible strides   -> tcgen05 kernel (gemm_tc.cu), tensor-core roofline
//   * bf16 / fp16, at most 8 rows per batch (decode attention: q*K^T and p*V over the KV cache)
//                                                        -> skinny kernels below: B is streamed once with 16-byte
//                                                           loads, HBM roofline, algorithmic bytes = bytes(B)
//   * everything else (fp32 / fp64 / odd strides)         -> SIMT tile kernel, exact fp32 (fp64) accumulation
#include "gemm.h"

#include "copy.h"
#include "device_utils.cuh"
#include "diopi/functions_b200.h"

namespace b200 {
namespace {

// ---- SIMT tile kernel (any float dtype, any strides) ---------------------------------------------------------------
struct SimtParams {
    int64_t batch, M, N, K;
    const void* A; int64_t a_sb, a_sm, a_sk;
    const void* B; int64_t b_sb, b_sk, b_sn;
    void* C; int64_t c_sb, c_sm, c_sn;
    const void* bias; int64_t bias_sb, bias_sm, bias_sn;
    diopiDtype_t a_dt, b_dt, c_dt, bias_dt;
    double alpha, beta;
};

template <typename Acc>
__global__ void __launch_bounds__(256) gemm_simt_kernel(const SimtParams p) {
    constexpr int TM = 64, TN = 64, TK = 16;
    __shared__ Acc sa[TK][TM + 1];
    __shared__ Acc sb[TK][TN + 1];
    const int64_t b = blockIdx.z;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * TM, n0 = static_cast<int64_t>(blockIdx.x) * TN;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    Acc acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = Acc(0);
    const char* Ab = static_cast<const char*>(p.A);
    const char* Bb = static_cast<const char*>(p.B);
    (void)Ab; (void)Bb;
    for (int64_t k0 = 0; k0 < p.K; k0 += TK) {
        for (int i = threadIdx.x; i < TM * TK; i += 256) {
            const int kk = i % TK, mm = i / TK;
            const int64_t m = m0 + mm, k = k0 + kk;
            sa[kk][mm] = (m < p.M && k < p.K) ? load_as<Acc>(p.A, p.a_dt, b * p.a_sb + m * p.a_sm + k * p.a_sk) : Acc(0);
        }
        for (int i = threadIdx.x; i < TN * TK; i += 256) {
            const int nn = i % TN, kk = i / TN;
            const int64_t n = n0 + nn, k = k0 + kk;
            sb[kk][nn] = (n < p.N && k < p.K) ? load_as<Acc>(p.B, p.b_dt, b * p.b_sb + k * p.b_sk + n * p.b_sn) : Acc(0);
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            Acc av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = sb[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] += av[i] * bv[j];
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int64_t m = m0 + ty * 4 + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t n = n0 + tx * 4 + j;
            if (n >= p.N) continue;
            Acc v = static_cast<Acc>(p.alpha) * acc[i][j];
            if (p.bias != nullptr) v += static_cast<Acc>(p.beta) * load_as<Acc>(p.bias, p.bias_dt, b * p.bias_sb + m * p.bias_sm + n * p.bias_sn);
            store_from<Acc>(p.C, p.c_dt, b * p.c_sb + m * p.c_sm + n * p.c_sn, v);
        }
    }
}

// ---- skinny kernels (M <= 8 rows per batch, 2-byte floats) --------------------------------------------------------------
constexpr int kSkinnyMaxM = 8;

struct SkinnyParams {
    int64_t batch, N, K;
    int M;
    const void* A; int64_t a_sb, a_sm;   // K contiguous
    const void* B; int64_t b_sb, b_ld;   // b_ld: pitch of the non-contiguous dim
    void* C; int64_t c_sb, c_sm;         // N contiguous
    float alpha;
};

// B is [batch, N, K] with K contiguous: every output is a dot product of a B row with an A row.
// A group of LPR lanes owns a B row (LPR * 8 elements per step); four rows are in flight per group.
template <typename T, int M_>
__global__ void __launch_bounds__(256) skinny_kmajor_kernel(const SkinnyParams p, int lpr) {
    const int lane = threadIdx.x & 31;
    const int gl = lane % lpr;                 // lane inside its group
    const int groups_per_warp = 32 / lpr;
    const int64_t group = (static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5)) * groups_per_warp + lane / lpr;
    const int64_t ngroups = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5) * groups_per_warp;
    const int64_t b = blockIdx.y;
    const T* A = static_cast<const T*>(p.A) + b * p.a_sb;
    const T* B = static_cast<const T*>(p.B) + b * p.b_sb;
    T* C = static_cast<T*>(p.C) + b * p.c_sb;
    constexpr int R = 4;  // B rows in flight per lane group (8 was measured slower: register pressure)
    const int64_t kvec = p.K / 8;
    // Every lane of the warp runs the same number of iterations so that the shuffles below stay warp-uniform.
    const int64_t nblocks = (p.N + R - 1) / R;
    const int64_t iters = (nblocks + ngroups - 1) / ngroups;
    for (int64_t it = 0; it < iters; ++it) {
        const int64_t n0 = (it * ngroups + group) * R;
        float acc[R][M_];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int m = 0; m < M_; ++m) acc[r][m] = 0.f;
        for (int64_t kv = gl; kv < kvec; kv += lpr) {
            Vec16<T> bv[R];
#pragma unroll
            for (int r = 0; r < R; ++r) {
                if (n0 + r < p.N) bv[r] = ld16_stream(B + (n0 + r) * p.b_ld + kv * 8);
            }
#pragma unroll
            for (int m = 0; m < M_; ++m) {
                const Vec16<T> av = ld16(A + m * p.a_sm + kv * 8);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (n0 + r < p.N) {
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r][m] += to_f32(av.v[e]) * to_f32(bv[r].v[e]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
            for (int m = 0; m < M_; ++m) {
                float v = acc[r][m];
                for (int o = lpr >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (gl == 0 && n0 + r < p.N) C[m * p.c_sm + n0 + r] = from_f32<T>(v * p.alpha);
            }
        }
    }
}

// B is [batch, K, N] with N contiguous. A thread owns 8 consecutive columns; the CTA's threads are arranged as
// (N/8 column groups) x (K splits) and the K splits are summed through shared memory.
template <typename T, int M_>
__global__ void __launch_bounds__(256) skinny_nmajor_kernel(const SkinnyParams p, int col_groups) {
    extern __shared__ float red[];  // [ksplit][M_][col_groups * 8]
    const int ksplit = blockDim.x / col_groups;
    const int cg = threadIdx.x % col_groups;
    const int ks = threadIdx.x / col_groups;
    const int64_t b = blockIdx.y;
    const int64_t n0 = (static_cast<int64_t>(blockIdx.x) * col_groups + cg) * 8;
    const T* A = static_cast<const T*>(p.A) + b * p.a_sb;
    const T* B = static_cast<const T*>(p.B) + b * p.b_sb;
    T* C = static_cast<T*>(p.C) + b * p.c_sb;
    float acc[M_][8];
#pragma unroll
    for (int m = 0; m < M_; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[m][e] = 0.f;
    if (n0 < p.N) {
        constexpr int U = 4;
        for (int64_t k0 = ks; k0 < p.K; k0 += static_cast<int64_t>(ksplit) * U) {
            Vec16<T> bv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t k = k0 + static_cast<int64_t>(u) * ksplit;
                if (k < p.K) bv[u] = ld16_stream(B + k * p.b_ld + n0);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t k = k0 + static_cast<int64_t>(u) * ksplit;
                if (k < p.K) {
#pragma unroll
                    for (int m = 0; m < M_; ++m) {
                        const float a = to_f32(A[m * p.a_sm + k]);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[m][e] += a * to_f32(bv[u].v[e]);
                    }
                }
            }
        }
    }
    const int width = col_groups * 8;
#pragma unroll
    for (int m = 0; m < M_; ++m)
#pragma unroll
        for (int e = 0; e < 8; ++e) red[(ks * M_ + m) * width + cg * 8 + e] = acc[m][e];
    __syncthreads();
    for (int i = threadIdx.x; i < M_ * width; i += blockDim.x) {
        const int m = i / width, c = i % width;
        const int64_t n = static_cast<int64_t>(blockIdx.x) * width + c;
        if (n < p.N) {
            float v = 0.f;
            for (int s = 0; s < ksplit; ++s) v += red[(s * M_ + m) * width + c];
            C[m * p.c_sm + n] = from_f32<T>(v * p.alpha);
        }
    }
}

template <typename T>
bool launch_skinny(const GemmProblem& g, cudaStream_t stream) {
    SkinnyParams p;
    p.batch = g.batch; p.N = g.N; p.K = g.K; p.M = static_cast<int>(g.M);
    p.A = g.A; p.a_sb = g.a_sb; p.a_sm = g.a_sm;
    p.B = g.B; p.b_sb = g.b_sb;
    p.C = g.C; p.c_sb = g.c_sb; p.c_sm = g.c_sm;
    p.alpha = g.alpha;
    const bool kmajor = g.b_sk == 1;
    p.b_ld = kmajor ? g.b_sn : g.b_sk;
#define SKINNY_M(KERNEL, GRID, BLOCK, SMEM, ARG)                                              \
    switch (p.M) {                                                                            \
        case 1: KERNEL<T, 1><<<GRID, BLOCK, SMEM, stream>>>(p, ARG); break;                   \
        case 2: KERNEL<T, 2><<<GRID, BLOCK, SMEM, stream>>>(p, ARG); break;                   \
        case 3: case 4: p.M = 4; KERNEL<T, 4><<<GRID, BLOCK, SMEM, stream>>>(p, ARG); break;  \
        default: p.M = 8; KERNEL<T, 8><<<GRID, BLOCK, SMEM, stream>>>(p, ARG); break;         \
    }
    // Row counts 3 and 5..7 would read rows of A and write rows of C that do not exist: those go elsewhere.
    if (!(g.M == 1 || g.M == 2 || g.M == 4 || g.M == 8)) return false;
    if (g.batch > 65535) return false;
    if (kmajor) {
        int lpr = 32;
        while (lpr > 1 && lpr * 8 > g.K) lpr >>= 1;
        const int groups_per_cta = 8 * (32 / lpr);
        const int rows_per_group = 4;
        int64_t bx = (g.N + rows_per_group * groups_per_cta - 1) / (rows_per_group * groups_per_cta);
        const int64_t cap = (static_cast<int64_t>(sm_count()) * 16 + g.batch - 1) / g.batch;
        if (bx > cap) bx = cap;
        if (bx < 1) bx = 1;
        dim3 grid(static_cast<unsigned>(bx), static_cast<unsigned>(g.batch));
        SKINNY_M(skinny_kmajor_kernel, grid, 256, 0, lpr)
    } else {
        int col_groups = 16;  // 128 columns per CTA
        while (col_groups > 1 && static_cast<int64_t>(col_groups) * 8 > g.N * 2) col_groups >>= 1;
        const int width = col_groups * 8;
        dim3 grid(static_cast<unsigned>((g.N + width - 1) / width), static_cast<unsigned>(g.batch));
        const int ksplit = 256 / col_groups;
        const int m_pad = p.M <= 2 ? p.M : (p.M <= 4 ? 4 : 8);
        const size_t smem = static_cast<size_t>(ksplit) * m_pad * width * sizeof(float);
        if (smem > 48 * 1024) return false;
        SKINNY_M(skinny_nmajor_kernel, grid, 256, smem, col_groups)
    }
#undef SKINNY_M
    return true;
}

bool skinny_eligible(const GemmProblem& g) {
    if (!(g.ab_dtype == diopi_dtype_bfloat16 || g.ab_dtype == diopi_dtype_float16) || g.c_dtype != g.ab_dtype) return false;
    if (!(g.M == 1 || g.M == 2 || g.M == 4 || g.M == 8) || g.bias != nullptr || g.batch > 65535) return false;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (g.a_sk != 1 || g.c_sn != 1 || !al16(g.B) || (g.b_sb % 8) != 0) return false;
    if (g.b_sk == 1) {
        // A rows are read as 16-byte vectors
        if (!al16(g.A) || (g.a_sb % 8) != 0 || (g.M > 1 && (g.a_sm % 8) != 0)) return false;
        return g.K % 8 == 0 && g.b_sn % 8 == 0;
    }
    if (g.b_sn == 1) return g.N % 8 == 0 && g.b_sk % 8 == 0;  // A is read element-wise here
    return false;
}

diopiError_t run_gemm(diopiContextHandle_t ctx, const char* name, const GemmProblem& g) {
    if (g.batch == 0 || g.M == 0 || g.N == 0) return diopiSuccess;
    cudaStream_t stream = stream_of(ctx);
    // Few-row products (decode attention over the KV cache) are bandwidth-bound either way; the tensor-core kernel is
    // tried first because its TMA pipeline streams B faster than per-thread loads do (measured 82 % / 103 % of the copy
    // bandwidth for q*K^T / p*V at batch 64, cache length 4096, against 72 % / 63 % for the kernels below). The skinny
    // kernels serve operands that do not meet the TMA alignment rules.
    if (g.K > 0 && gemm_tc_eligible(g)) return gemm_tc_launch(g, stream);
    if (g.K > 0 && skinny_eligible(g)) {
        bool ok = (g.ab_dtype == diopi_dtype_bfloat16) ? launch_skinny<bf16>(g, stream) : launch_skinny<fp16>(g, stream);
        if (ok) {
            B200_LAUNCH_CHECK(name);
            return diopiSuccess;
        }
    }
    B200_CHECK(is_floating(g.ab_dtype) && is_floating(g.c_dtype), "%s: only floating dtypes are supported (got %s -> %s)", name,
               dtype_name(g.ab_dtype), dtype_name(g.c_dtype));
    B200_CHECK(g.batch <= 65535, "%s: batch %lld too large for the general kernel", name, (long long)g.batch);
    SimtParams p;
    p.batch = g.batch; p.M = g.M; p.N = g.N; p.K = g.K;
    p.A = g.A; p.a_sb = g.a_sb; p.a_sm = g.a_sm; p.a_sk = g.a_sk;
    p.B = g.B; p.b_sb = g.b_sb; p.b_sk = g.b_sk; p.b_sn = g.b_sn;
    p.C = g.C; p.c_sb = g.c_sb; p.c_sm = g.c_sm; p.c_sn = g.c_sn;
    p.bias = g.bias; p.bias_sb = g.bias_sb; p.bias_sm = g.bias_sm; p.bias_sn = g.bias_sn;
    p.a_dt = g.ab_dtype; p.b_dt = g.ab_dtype; p.c_dt = g.c_dtype; p.bias_dt = g.bias_dtype;
    p.alpha = g.alpha; p.beta = g.beta;
    dim3 grid(static_cast<unsigned>((g.N + 63) / 64), static_cast<unsigned>((g.M + 63) / 64), static_cast<unsigned>(g.batch));
    B200_CHECK(grid.y <= 65535, "%s: M too large for the general kernel", name);
    if (g.c_dtype == diopi_dtype_float64 || g.ab_dtype == diopi_dtype_float64) gemm_simt_kernel<double><<<grid, 256, 0, stream>>>(p);
    else gemm_simt_kernel<float><<<grid, 256, 0, stream>>>(p);
    B200_LAUNCH_CHECK(name);
    return diopiSuccess;
}

// Fills bias strides for a tensor that must broadcast to [batch, M, N].
bool set_bias(GemmProblem* g, const TensorView& vb, bool batched) {
    const int want = batched ? 3 : 2;
    if (vb.ndim > want) return false;
    int64_t shp[3] = {1, 1, 1}, str[3] = {0, 0, 0};
    for (int d = 0; d < vb.ndim; ++d) {
        shp[3 - vb.ndim + d] = vb.shape[d];
        str[3 - vb.ndim + d] = vb.stride[d];
    }
    const int64_t want_shape[3] = {g->batch, g->M, g->N};
    for (int d = 0; d < 3; ++d) {
        if (shp[d] == want_shape[d]) { if (shp[d] == 1) str[d] = 0; }
        else if (shp[d] == 1) str[d] = 0;
        else return false;
    }
    g->bias = vb.data; g->bias_sb = str[0]; g->bias_sm = str[1]; g->bias_sn = str[2];
    g->bias_dtype = vb.dtype;
    return true;
}

double scalar_as_double(const diopiScalar_t* s, double dflt) {
    if (s == nullptr) return dflt;
    return (s->stype == diopi_dtype_float64 || s->stype == diopi_dtype_float32) ? s->fval : static_cast<double>(s->ival);
}

diopiError_t mm_like(diopiContextHandle_t ctx, const char* name, const TensorView& vo, const TensorView& va, const TensorView& vb,
                     const TensorView* bias, double alpha, double beta, bool batched) {
    const int nd = batched ? 3 : 2;
    B200_CHECK(va.ndim == nd && vb.ndim == nd && vo.ndim == nd, "%s: expected %d-d operands (got %d, %d -> %d)", name, nd, va.ndim, vb.ndim, vo.ndim);
    B200_CHECK(va.device == diopi_device && vb.device == diopi_device && vo.device == diopi_device, "%s: operands must be device tensors", name);
    B200_CHECK(va.dtype == vb.dtype, "%s: operand dtypes differ (%s vs %s)", name, dtype_name(va.dtype), dtype_name(vb.dtype));
    const int o = batched ? 1 : 0;
    GemmProblem g;
    g.batch = batched ? va.shape[0] : 1;
    g.M = va.shape[o]; g.K = va.shape[o + 1]; g.N = vb.shape[o + 1];
    B200_CHECK(vb.shape[o] == g.K, "%s: inner dimensions differ (%lld vs %lld)", name, (long long)g.K, (long long)vb.shape[o]);
    B200_CHECK(vo.shape[o] == g.M && vo.shape[o + 1] == g.N, "%s: output shape mismatch", name);
    if (batched) B200_CHECK(vb.shape[0] == g.batch && vo.shape[0] == g.batch, "%s: batch sizes differ", name);
    g.A = va.data; g.a_sb = batched ? va.stride[0] : 0; g.a_sm = va.stride[o]; g.a_sk = va.stride[o + 1];
    g.B = vb.data; g.b_sb = batched ? vb.stride[0] : 0; g.b_sk = vb.stride[o]; g.b_sn = vb.stride[o + 1];
    g.C = vo.data; g.c_sb = batched ? vo.stride[0] : 0; g.c_sm = vo.stride[o]; g.c_sn = vo.stride[o + 1];
    // size-1 dims carry arbitrary strides: give them the dense value so the layout tests below see what matters
    if (g.K == 1) g.a_sk = 1;
    if (g.M == 1) {
        if (g.a_sk == 1) g.a_sm = g.K;
        if (g.c_sn == 1 || g.N == 1) g.c_sm = g.N;
    }
    if (g.N == 1) {
        g.c_sn = 1;
        if (g.b_sk == 1) g.b_sn = g.K; else g.b_sn = 1;
    }
    g.ab_dtype = va.dtype; g.c_dtype = vo.dtype;
    g.alpha = static_cast<float>(alpha); g.beta = static_cast<float>(beta);
    if (bias != nullptr && beta != 0.0) {
        B200_CHECK(set_bias(&g, *bias, batched), "%s: the additive input cannot be broadcast to the output", name);
    }
    if (g.K == 0) {
        // empty inner dimension: the product is all zeros
        B200_CHECK(bias == nullptr || beta == 0.0, "%s: K == 0 with an additive input is not supported", name);
    }
    return run_gemm(ctx, name, g);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

diopiError_t diopiMm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat2) {
    B200_VIEW(vo, out);
    B200_VIEW(va, input);
    B200_VIEW(vb, mat2);
    return mm_like(ctx, "diopiMm", vo, va, vb, nullptr, 1.0, 0.0, false);
}

// out [M, F] = silu(input x gate columns) * (input x up columns) for mat2 [K, 2F] whose columns 2j / 2j+1 are the gate / up
// weights of feature j: one product over the interleaved weight with the SiLU and the multiplication in its epilogue.
diopiError_t diopiB200MmSwiGLU(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat2) {
    B200_VIEW(vo, out);
    B200_VIEW(va, input);
    B200_VIEW(vb, mat2);
    B200_CHECK(va.ndim == 2 && vb.ndim == 2 && vo.ndim == 2 && va.shape[1] == vb.shape[0], "diopiB200MmSwiGLU: expected [M, K] x [K, 2F] -> [M, F]");
    B200_CHECK(vb.shape[1] % 2 == 0 && vo.shape[0] == va.shape[0] && vo.shape[1] * 2 == vb.shape[1], "diopiB200MmSwiGLU: output must be [M, F] for mat2 [K, 2F]");
    B200_CHECK(va.device == diopi_device && vb.device == diopi_device && vo.device == diopi_device, "diopiB200MmSwiGLU: operands must be device tensors");
    B200_CHECK(va.dtype == vb.dtype && vo.dtype == va.dtype && (va.dtype == diopi_dtype_bfloat16 || va.dtype == diopi_dtype_float16),
               "diopiB200MmSwiGLU: bfloat16 or float16 tensors of one dtype");
    B200_CHECK(va.shape[0] >= 1 && va.shape[0] <= 128, "diopiB200MmSwiGLU: served for 1 to 128 rows (decode batches); got %lld", (long long)va.shape[0]);
    B200_CHECK(vo.stride[1] == 1 && vo.stride[0] >= vo.shape[1], "diopiB200MmSwiGLU: output rows must be contiguous");
    GemmProblem g;
    g.M = va.shape[0]; g.K = va.shape[1]; g.N = vb.shape[1];
    g.A = va.data; g.a_sm = va.stride[0]; g.a_sk = va.stride[1];
    g.B = vb.data; g.b_sk = vb.stride[0]; g.b_sn = vb.stride[1];
    g.C = vo.data; g.c_sm = vo.stride[0]; g.c_sn = 1;
    g.ab_dtype = va.dtype; g.c_dtype = vo.dtype;
    g.epilogue = GemmProblem::kSwiGLU;
    GemmProblem operands = g;   // the layout rules concern the operands; the output is half as wide as the product
    operands.c_sm = g.c_sm >= g.N ? g.c_sm : g.N;
    B200_CHECK(gemm_tc_eligible(operands), "diopiB200MmSwiGLU: operands do not meet the tensor-core kernel's layout rules (16-byte aligned pointers, "
               "pitches that are multiples of 8 elements, K or N contiguous)");
    return gemm_tc_launch(g, stream_of(ctx));
}

// mat1 [M, K] x mat2 [K, N]: this rank's partial sum of a row-parallel linear, pushed into the peers' staging slots.
diopiError_t diopiB200MmPush(diopiContextHandle_t ctx, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat2, const b200PeerSpace* space,
                             int32_t slot, uint32_t epoch, uint32_t prev_epoch) {
    B200_CHECK(space != nullptr, "diopiB200MmPush: NULL peer space");
    B200_VIEW(va, input);
    B200_VIEW(vb, mat2);
    B200_CHECK(va.ndim == 2 && vb.ndim == 2 && va.shape[1] == vb.shape[0], "diopiB200MmPush: expected [M, K] x [K, N]");
    B200_CHECK(va.device == diopi_device && vb.device == diopi_device, "diopiB200MmPush: operands must be device tensors");
    B200_CHECK(va.dtype == vb.dtype && (va.dtype == diopi_dtype_bfloat16 || va.dtype == diopi_dtype_float16),
               "diopiB200MmPush: operands must both be bfloat16 or float16");
    GemmProblem g;
    g.M = va.shape[0]; g.K = va.shape[1]; g.N = vb.shape[1];
    g.A = va.data; g.a_sm = va.stride[0]; g.a_sk = va.stride[1];
    g.B = vb.data; g.b_sk = vb.stride[0]; g.b_sn = vb.stride[1];
    g.C = nullptr; g.c_sm = g.N; g.c_sn = 1;
    g.ab_dtype = va.dtype; g.c_dtype = va.dtype;
    B200_CHECK(gemm_tc_eligible(g), "diopiB200MmPush: operands do not meet the tensor-core kernel's layout rules (16-byte aligned pointers, pitches "
               "that are multiples of 8 elements, K or N contiguous)");
    return gemm_tc2_push_launch(g, *space, slot, epoch, prev_epoch, stream_of(ctx));
}

diopiError_t diopiAddmm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat1,
                        diopiConstTensorHandle_t mat2, const diopiScalar_t* beta, const diopiScalar_t* alpha) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_VIEW(va, mat1);
    B200_VIEW(vb, mat2);
    return mm_like(ctx, "diopiAddmm", vo, va, vb, &vi, scalar_as_double(alpha, 1.0), scalar_as_double(beta, 1.0), false);
}

diopiError_t diopiBmm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t mat2) {
    B200_VIEW(vo, out);
    B200_VIEW(va, input);
    B200_VIEW(vb, mat2);
    return mm_like(ctx, "diopiBmm", vo, va, vb, nullptr, 1.0, 0.0, true);
}

diopiError_t diopiBaddbmm(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t batch1,
                          diopiConstTensorHandle_t batch2, double beta, double alpha) {
    B200_VIEW(vo, out);
    B200_VIEW(vi, input);
    B200_VIEW(va, batch1);
    B200_VIEW(vb, batch2);
    return mm_like(ctx, "diopiBaddbmm", vo, va, vb, &vi, alpha, beta, true);
}

diopiError_t diopiBaddbmmInp(diopiContextHandle_t ctx, diopiTensorHandle_t input, diopiConstTensorHandle_t batch1, diopiConstTensorHandle_t batch2,
                             double beta, double alpha) {
    return diopiBaddbmm(ctx, input, input, batch1, batch2, beta, alpha);
}

diopiError_t diopiLinear(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t weight,
                         diopiConstTensorHandle_t bias) {
    B200_VIEW(vo, out);
    B200_VIEW(vi_raw, input);
    B200_VIEW(vw, weight);
    B200_CHECK(vw.ndim == 2 && vi_raw.ndim >= 1, "diopiLinear: weight must be 2-d");
    TensorView vi;
    if (make_contiguous(ctx, vi_raw, &vi) != diopiSuccess) return diopiErrorOccurred;
    B200_CHECK(vo.is_contiguous(), "diopiLinear: output must be contiguous");
    const int64_t K = vw.shape[1], N = vw.shape[0];
    B200_CHECK(vi.shape[vi.ndim - 1] == K, "diopiLinear: input features %lld != weight in-features %lld", (long long)vi.shape[vi.ndim - 1], (long long)K);
    // fold all leading dims into rows; the weight is used through its transposed view
    TensorView a2 = vi, o2 = vo, wt = vw;
    a2.ndim = 2; a2.shape[0] = vi.numel / K; a2.shape[1] = K; a2.stride[0] = K; a2.stride[1] = 1;
    o2.ndim = 2; o2.shape[0] = vo.numel / N; o2.shape[1] = N; o2.stride[0] = N; o2.stride[1] = 1;
    wt.shape[0] = K; wt.shape[1] = N; wt.stride[0] = vw.stride[1]; wt.stride[1] = vw.stride[0];
    if (bias != nullptr) {
        B200_VIEW(vbias, bias);
        return mm_like(ctx, "diopiLinear", o2, a2, wt, &vbias, 1.0, 1.0, false);
    }
    return mm_like(ctx, "diopiLinear", o2, a2, wt, nullptr, 1.0, 0.0, false);
}

// torch.matmul semantics for the shapes DIPU's adapter forwards: 1-d/2-d combinations and N-d x {1,2,N}-d with
// broadcast batch dims. Batched cases are reduced to one bmm over a folded batch dimension.
diopiError_t diopiMatmul(diopiContextHandle_t ctx, diopiTensorHandle_t out, diopiConstTensorHandle_t input, diopiConstTensorHandle_t other) {
    B200_VIEW(vo, out);
    B200_VIEW(va_raw, input);
    B200_VIEW(vb_raw, other);
    B200_CHECK(va_raw.ndim >= 1 && vb_raw.ndim >= 1, "diopiMatmul: operands must have at least one dimension");
    B200_CHECK(vo.is_contiguous(), "diopiMatmul: output must be contiguous");
    TensorView a = va_raw, b = vb_raw;
    // promote vectors to matrices
    if (a.ndim == 1) { a.ndim = 2; a.shape[1] = a.shape[0]; a.stride[1] = a.stride[0]; a.shape[0] = 1; a.stride[0] = 0; }
    if (b.ndim == 1) { b.ndim = 2; b.shape[1] = 1; b.stride[1] = 0; }
    const int64_t M = a.shape[a.ndim - 2], K = a.shape[a.ndim - 1], N = b.shape[b.ndim - 1];
    B200_CHECK(b.shape[b.ndim - 2] == K, "diopiMatmul: inner dimensions differ");
    // batch shape = broadcast of leading dims
    const int nba = a.ndim - 2, nbb = b.ndim - 2, nb = nba > nbb ? nba : nbb;
    int64_t bshape[kMaxDims], bsa[kMaxDims], bsb[kMaxDims];
    int64_t batch = 1;
    for (int d = 0; d < nb; ++d) {
        const int ia = d - (nb - nba), ib = d - (nb - nbb);
        const int64_t sa = ia >= 0 ? a.shape[ia] : 1, sb = ib >= 0 ? b.shape[ib] : 1;
        B200_CHECK(sa == sb || sa == 1 || sb == 1, "diopiMatmul: batch dimensions cannot be broadcast");
        bshape[d] = sa > sb ? sa : sb;
        bsa[d] = (ia >= 0 && sa != 1) ? a.stride[ia] : 0;
        bsb[d] = (ib >= 0 && sb != 1) ? b.stride[ib] : 0;
        batch *= bshape[d];
    }
    B200_CHECK(vo.numel == batch * M * N, "diopiMatmul: output has %lld elements, expected %lld", (long long)vo.numel, (long long)(batch * M * N));
    // A [*, M, K] x B [K, N] with foldable leading dims of A -> one plain mm over (batch*M) rows
    bool b_bcast = true;
    for (int d = 0; d < nb; ++d) b_bcast = b_bcast && bsb[d] == 0;
    if (nb > 0 && b_bcast) {
        TensorView ac;
        if (make_contiguous(ctx, a, &ac) != diopiSuccess) return diopiErrorOccurred;
        TensorView a2 = ac, o2 = vo, b2 = b;
        a2.ndim = 2; a2.shape[0] = batch * M; a2.shape[1] = K; a2.stride[0] = K; a2.stride[1] = 1;
        o2.ndim = 2; o2.shape[0] = batch * M; o2.shape[1] = N; o2.stride[0] = N; o2.stride[1] = 1;
        b2.ndim = 2; b2.shape[0] = K; b2.shape[1] = N; b2.stride[0] = b.stride[b.ndim - 2]; b2.stride[1] = b.stride[b.ndim - 1];
        return mm_like(ctx, "diopiMatmul", o2, a2, b2, nullptr, 1.0, 0.0, false);
    }
    // general: fold the batch dims into one; needs a uniform batch stride per operand -> densify when it is not
    auto fold = [&](const TensorView& t, const int64_t* bs, int64_t* sb_out, TensorView* folded) -> diopiError_t {
        // uniform if strides nest: bs[d] == bs[d+1] * bshape[d+1] for all d (or all zero)
        bool uniform = true;
        for (int d = 0; d + 1 < nb; ++d) uniform = uniform && (bs[d] == bs[d + 1] * bshape[d + 1]);
        if (uniform) {
            *folded = t;
            *sb_out = nb > 0 ? bs[nb - 1] : 0;
            return diopiSuccess;
        }
        // materialise the broadcast batch view densely
        TensorView expanded = t;
        expanded.ndim = nb + 2;
        for (int d = 0; d < nb; ++d) { expanded.shape[d] = bshape[d]; expanded.stride[d] = bs[d]; }
        expanded.shape[nb] = t.shape[t.ndim - 2]; expanded.stride[nb] = t.stride[t.ndim - 2];
        expanded.shape[nb + 1] = t.shape[t.ndim - 1]; expanded.stride[nb + 1] = t.stride[t.ndim - 1];
        expanded.numel = batch * expanded.shape[nb] * expanded.shape[nb + 1];
        diopiTensorHandle_t tmp = nullptr;
        diopiSize_t size{expanded.shape, expanded.ndim};
        B200_CHECK(diopiRequireTensor(ctx, &tmp, &size, nullptr, t.dtype, diopi_device) == diopiSuccess && tmp != nullptr, "diopiMatmul: workspace allocation failed");
        if (!make_view(tmp, folded, "workspace")) return diopiErrorOccurred;
        if (copy_impl(ctx, expanded, *folded) != diopiSuccess) return diopiErrorOccurred;
        *sb_out = folded->shape[nb] * folded->shape[nb + 1];
        return diopiSuccess;
    };
    TensorView fa, fb;
    int64_t sba = 0, sbb = 0;
    if (fold(a, bsa, &sba, &fa) != diopiSuccess) return diopiErrorOccurred;
    if (fold(b, bsb, &sbb, &fb) != diopiSuccess) return diopiErrorOccurred;
    TensorView a3 = fa, b3 = fb, o3 = vo;
    a3.ndim = 3; a3.shape[0] = batch; a3.shape[1] = M; a3.shape[2] = K;
    a3.stride[0] = sba; a3.stride[1] = fa.stride[fa.ndim - 2]; a3.stride[2] = fa.stride[fa.ndim - 1];
    b3.ndim = 3; b3.shape[0] = batch; b3.shape[1] = K; b3.shape[2] = N;
    b3.stride[0] = sbb; b3.stride[1] = fb.stride[fb.ndim - 2]; b3.stride[2] = fb.stride[fb.ndim - 1];
    o3.ndim = 3; o3.shape[0] = batch; o3.shape[1] = M; o3.shape[2] = N; o3.stride[0] = M * N; o3.stride[1] = N; o3.stride[2] = 1;
    return mm_like(ctx, "diopiMatmul", o3, a3, b3, nullptr, 1.0, 0.0, true);
}

}  // extern "C"
