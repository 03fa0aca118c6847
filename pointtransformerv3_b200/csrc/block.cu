// One call per transformer block (model.py:519-606, inference, pre-norm):
//
//     x    = SubMConv3d(conv_in)                               xCPE convolution
//     f1   = feat + LN_cpe(Linear_cpe(x));  a = LN_1(f1)
//     qkv  = Linear_qkv(a);  att = patch attention(qkv)
//     f2   = f1 + Linear_proj(att);         b = LN_2(f2)
//     out  = f2 + fc2(GELU(fc1(b)))
//
// The kernels are the ones behind the single-operator entry points; this file
// only queues them back to back from C++, so that a block costs the host one
// call instead of a dozen (on the coarse levels, where every kernel runs for a
// few microseconds, the Python-side cost of a launch is what bounds the step).
// Channel widths the tcgen05 kernels cover (32, 64, 128) use them; wider blocks
// take their Linear layers from cuBLASLt (plain library GEMMs with a bias
// epilogue) and the LayerNorm / residual glue from the fused row kernel.
#include <cublasLt.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "vec.cuh"

namespace ptv3 {

// ---------------------------------------------------------------------------
// cuBLASLt: out[n x n_out] = x[n x k] W^T + b, bf16 operands, fp32 accumulation
// ---------------------------------------------------------------------------
namespace {

struct GemmPlan {
    cublasLtMatmulDesc_t op = nullptr;
    cublasLtMatrixLayout_t a = nullptr, b = nullptr, c = nullptr;
    cublasLtMatmulAlgo_t algo;
    bool ok = false;
};

struct GemmCache {
    std::mutex mu;
    cublasLtHandle_t handle = nullptr;
    std::map<std::tuple<int, int64_t, int, int, size_t>, GemmPlan> plans;   // device, n, k, n_out, workspace
};

GemmCache& gemm_cache()
{
    static GemmCache c;
    return c;
}

#define PTV3_LT(call)                                                                   \
    do {                                                                                \
        const cublasStatus_t st_ = (call);                                              \
        if (st_ != CUBLAS_STATUS_SUCCESS) {                                             \
            set_error("cuBLASLt: %s failed with status %d", #call, (int)st_);           \
            return PTV3_ERR_CUDA;                                                       \
        }                                                                               \
    } while (0)

int build_plan(cublasLtHandle_t handle, int64_t n, int k, int n_out, size_t ws_bytes, GemmPlan* p)
{
    // row-major out = x W^T is column-major out^T (n_out x n) = W^T-as-stored (k x n_out)^T . x^T (k x n)
    const cublasOperation_t ta = CUBLAS_OP_T, tb = CUBLAS_OP_N;
    const cublasLtEpilogue_t epi = CUBLASLT_EPILOGUE_BIAS;
    const cudaDataType_t bf16 = CUDA_R_16BF;
    PTV3_LT(cublasLtMatmulDescCreate(&p->op, CUBLAS_COMPUTE_32F, CUDA_R_32F));
    PTV3_LT(cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_TRANSA, &ta, sizeof(ta)));
    PTV3_LT(cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_TRANSB, &tb, sizeof(tb)));
    PTV3_LT(cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_EPILOGUE, &epi, sizeof(epi)));
    PTV3_LT(cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_BIAS_DATA_TYPE, &bf16, sizeof(bf16)));
    PTV3_LT(cublasLtMatrixLayoutCreate(&p->a, bf16, (uint64_t)k, (uint64_t)n_out, k));
    PTV3_LT(cublasLtMatrixLayoutCreate(&p->b, bf16, (uint64_t)k, (uint64_t)n, k));
    PTV3_LT(cublasLtMatrixLayoutCreate(&p->c, bf16, (uint64_t)n_out, (uint64_t)n, n_out));
    // the bias pointer is part of the descriptor the heuristic sees; any non-null value does
    const void* probe = reinterpret_cast<const void*>(16);
    PTV3_LT(cublasLtMatmulDescSetAttribute(p->op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &probe, sizeof(probe)));
    cublasLtMatmulPreference_t pref = nullptr;
    PTV3_LT(cublasLtMatmulPreferenceCreate(&pref));
    PTV3_LT(cublasLtMatmulPreferenceSetAttribute(pref, CUBLASLT_MATMUL_PREF_MAX_WORKSPACE_BYTES, &ws_bytes,
                                                 sizeof(ws_bytes)));
    cublasLtMatmulHeuristicResult_t res;
    int found = 0;
    const cublasStatus_t st = cublasLtMatmulAlgoGetHeuristic(handle, p->op, p->a, p->b, p->c, p->c, pref, 1, &res,
                                                             &found);
    cublasLtMatmulPreferenceDestroy(pref);
    if (st != CUBLAS_STATUS_SUCCESS || found == 0) {
        set_error("cuBLASLt: no algorithm for a %lld x %d x %d bf16 GEMM (status %d)", (long long)n, k, n_out,
                  (int)st);
        return PTV3_ERR_UNSUPPORTED;
    }
    p->algo = res.algo;
    p->ok = true;
    return PTV3_OK;
}

}  // namespace

// `ws` is the caller's scratch for the library (may be null with ws_bytes 0)
static int gemm_bias_bf16(const void* x, const void* w, const void* bias, void* out, int64_t n, int k, int n_out,
                          void* ws, size_t ws_bytes, cudaStream_t stream)
{
    if (n == 0) return PTV3_OK;
    GemmCache& gc = gemm_cache();
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(gc.mu);
        if (!gc.handle) PTV3_LT(cublasLtCreate(&gc.handle));
        // row counts change with every batch in service: keep the table bounded
        if (gc.plans.size() >= 2048) {
            for (auto& kv : gc.plans) {
                if (kv.second.op) cublasLtMatmulDescDestroy(kv.second.op);
                if (kv.second.a) cublasLtMatrixLayoutDestroy(kv.second.a);
                if (kv.second.b) cublasLtMatrixLayoutDestroy(kv.second.b);
                if (kv.second.c) cublasLtMatrixLayoutDestroy(kv.second.c);
            }
            gc.plans.clear();
        }
        GemmPlan& p = gc.plans[std::make_tuple(dev, n, k, n_out, ws_bytes)];
        if (!p.ok) {
            const int rc = build_plan(gc.handle, n, k, n_out, ws_bytes, &p);
            if (rc != PTV3_OK) return rc;
        }
        // the bias pointer lives in the operation descriptor: set and launch under the lock
        PTV3_LT(cublasLtMatmulDescSetAttribute(p.op, CUBLASLT_MATMUL_DESC_BIAS_POINTER, &bias, sizeof(bias)));
        const float one = 1.f, zero = 0.f;
        PTV3_LT(cublasLtMatmul(gc.handle, p.op, &one, w, p.a, x, p.b, &zero, out, p.c, out, p.c, &p.algo, ws,
                               ws_bytes, stream));
    }
    count_launches(1);
    return PTV3_OK;
}

// exact GELU in place on bf16 (the bias was added by the GEMM epilogue)
__global__ void __launch_bounds__(256) gelu_bf16_kernel(__nv_bfloat16* __restrict__ x, int64_t n8)
{
    const int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i >= n8) return;
    uint4 v = reinterpret_cast<uint4*>(x)[i];
    uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[j]));
        f.x = 0.5f * f.x * (1.f + erff(f.x * 0.70710678f));
        f.y = 0.5f * f.y * (1.f + erff(f.y * 0.70710678f));
        const __nv_bfloat162 r = __floats2bfloat162_rn(f.x, f.y);
        w[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    reinterpret_cast<uint4*>(x)[i] = v;
}

static constexpr size_t BLOCK_LT_WORKSPACE = (size_t)32 << 20;

struct BlockBuffers {
    void *x, *f1, *a, *qkv, *att, *f2, *hidden, *acc32, *lt;
};

static size_t carve_block(const ptv3_block_args* a, void* base, BlockBuffers* b)
{
    const size_t row = (size_t)a->channels * 2;
    const size_t n = (size_t)a->n;
    const bool fused_mlp = ptv3_mlp_supported(a->channels, a->hidden, a->dtype) != 0;
    Carver c(base);
    BlockBuffers t;
    t.x = c.take<char>(n * row);
    t.f1 = c.take<char>(n * row);
    t.a = c.take<char>(n * row);
    t.qkv = c.take<char>(n * row * 3);
    t.att = t.x;   // the convolution output is dead once f1 exists
    t.f2 = c.take<char>(n * row);
    t.hidden = fused_mlp ? nullptr : c.take<char>(n * (size_t)a->hidden * 2);
    t.acc32 = a->pair_in ? c.take<char>(n * (size_t)a->channels * 8) : nullptr;
    t.lt = c.take<char>(BLOCK_LT_WORKSPACE);
    if (b) *b = t;
    return c.off;
}

}  // namespace ptv3

using namespace ptv3;

extern "C" int ptv3_block_supported(int channels, int heads, int hidden, int dtype)
{
    return dtype == PTV3_DTYPE_BF16 && heads > 0 && channels % heads == 0 && channels % 16 == 0 &&
           hidden % 16 == 0 && channels >= 16 && hidden >= 16;
}

extern "C" size_t ptv3_block_workspace_bytes(const ptv3_block_args* a)
{
    if (!a || a->n < 0) return 0;
    return carve_block(a, nullptr, nullptr);
}

extern "C" int ptv3_block_fwd(const ptv3_block_args* a, void* stream_)
{
    PTV3_REQUIRE(a != nullptr, PTV3_ERR_INVALID_ARGUMENT, "ptv3_block_fwd: null argument block");
    PTV3_REQUIRE(ptv3_block_supported(a->channels, a->heads, a->hidden, a->dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_block_fwd: bf16 only, channels and hidden multiples of 16 (got %d, %d, dtype %d)",
                 a->channels, a->hidden, a->dtype);
    PTV3_REQUIRE(a->n >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_block_fwd: n < 0");
    if (a->n == 0) return PTV3_OK;
    PTV3_REQUIRE(a->conv_in && a->feat && a->out && a->status && a->workspace && a->conv_weight && a->cpe_w &&
                     a->cpe_b && a->cpe_ln_w && a->cpe_ln_b && a->n1_w && a->n1_b && a->qkv_w && a->qkv_b &&
                     a->proj_w && a->proj_b && a->n2_w && a->n2_b && a->fc1_w && a->fc1_b && a->fc2_w &&
                     a->fc2_b && a->order && a->pad && a->unpad && a->cu_seqlens && (a->nbr || a->pair_in),
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_block_fwd: null pointer");
    PTV3_REQUIRE(a->workspace_bytes >= carve_block(a, nullptr, nullptr), PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_block_fwd: workspace of %zu bytes, %zu needed", a->workspace_bytes,
                 carve_block(a, nullptr, nullptr));
    cudaStream_t stream = (cudaStream_t)stream_;
    BlockBuffers b;
    carve_block(a, a->workspace, &b);
    const int C = a->channels, dt = a->dtype;
    const int64_t n = a->n;
    int rc;
#define STEP(call)               \
    do {                         \
        rc = (call);             \
        if (rc != PTV3_OK) return rc; \
    } while (0)

    // xCPE convolution
    if (a->pair_in)
        STEP(ptv3_subm_conv_pairs_fwd(a->conv_in, a->pair_in, a->pair_out, a->off_start, a->tile_start,
                                      a->conv_weight, a->conv_bias, b.x, b.acc32, (size_t)n * C * 8, n, C, C, 27,
                                      dt, stream_));
    else
        STEP(ptv3_subm_conv_fwd(a->conv_in, a->nbr, a->conv_weight, a->conv_bias, b.x, a->row_order, n, C, C, 27,
                                dt, 0, stream_));

    const bool tc_lin = ptv3_linear_supported(C, C, 1, dt) && ptv3_linear_supported(C, 3 * C, 0, dt);
    if (tc_lin) {
        STEP(ptv3_linear_ln_fwd(b.x, a->cpe_w, a->cpe_b, a->feat, a->cpe_ln_w, a->cpe_ln_b, a->cpe_ln_eps, b.f1,
                                a->n1_w, a->n1_b, a->n1_eps, b.a, n, C, dt, a->status, stream_));
        STEP(ptv3_linear_fwd(b.a, a->qkv_w, a->qkv_b, b.qkv, n, C, 3 * C, dt, a->status, stream_));
    } else {
        // library GEMM, then f1 = feat + LN_cpe(.), a = LN_1(f1) in the fused row kernel
        // (the qkv buffer is free here and serves as the GEMM's output)
        STEP(gemm_bias_bf16(b.x, a->cpe_w, a->cpe_b, b.qkv, n, C, C, b.lt, BLOCK_LT_WORKSPACE, stream));
        STEP(ptv3_add_layernorm_fwd(b.qkv, a->feat, a->cpe_ln_w, a->cpe_ln_b, a->cpe_ln_eps, b.f1, a->n1_w, a->n1_b,
                                    a->n1_eps, b.a, n, C, dt, stream_));
        STEP(gemm_bias_bf16(b.a, a->qkv_w, a->qkv_b, b.qkv, n, C, 3 * C, b.lt, BLOCK_LT_WORKSPACE, stream));
    }
    STEP(ptv3_attention_fwd(b.qkv, a->order, a->pad, a->unpad, a->cu_seqlens, b.att, n, a->n_seq, a->max_seqlen, C,
                            a->heads, a->scale, dt, a->attention_algo, a->status, stream_));
    const bool fused_mlp = ptv3_mlp_supported(C, a->hidden, dt) != 0;
    if (tc_lin) {
        STEP(ptv3_linear_ln_fwd(b.att, a->proj_w, a->proj_b, b.f1, nullptr, nullptr, 0.f, b.f2, a->n2_w, a->n2_b,
                                a->n2_eps, b.a, n, C, dt, a->status, stream_));
    } else {
        STEP(gemm_bias_bf16(b.att, a->proj_w, a->proj_b, b.qkv, n, C, C, b.lt, BLOCK_LT_WORKSPACE, stream));
        STEP(ptv3_add_layernorm_fwd(b.qkv, b.f1, nullptr, nullptr, 0.f, b.f2, a->n2_w, a->n2_b, a->n2_eps, b.a, n, C,
                                    dt, stream_));
    }
    if (fused_mlp) {
        STEP(ptv3_mlp_fwd(b.a, a->fc1_w, a->fc1_b, a->fc2_w, a->fc2_b, b.f2, a->out, n, C, a->hidden, dt, a->status,
                          stream_));
    } else {
        STEP(gemm_bias_bf16(b.a, a->fc1_w, a->fc1_b, b.hidden, n, C, a->hidden, b.lt, BLOCK_LT_WORKSPACE, stream));
        const int64_t n8 = n * a->hidden / 8;
        gelu_bf16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, stream>>>((__nv_bfloat16*)b.hidden, n8);
        count_launches(1);
        STEP(check_launch("ptv3_block_fwd: GELU"));
        STEP(gemm_bias_bf16(b.hidden, a->fc2_w, a->fc2_b, b.qkv, n, a->hidden, C, b.lt, BLOCK_LT_WORKSPACE, stream));
        // out = f2 + fc2(...)
        STEP(ptv3_add_layernorm_fwd(b.qkv, b.f2, nullptr, nullptr, 0.f, a->out, nullptr, nullptr, 0.f, nullptr, n, C,
                                    dt, stream_));
    }
#undef STEP
    return PTV3_OK;
}

// ---------------------------------------------------------------------------
// Stage transitions in one call each: the projection(s) by cuBLASLt followed by the
// pooling / unpooling kernel (model.py:684-689, 707-710 and model.py:726-735, 744-746).
// ---------------------------------------------------------------------------
extern "C" size_t ptv3_pool_stage_workspace_bytes(int64_t n, int c_out)
{
    if (n <= 0 || c_out <= 0) return 0;
    return align_up((size_t)n * c_out * 2, 256) + BLOCK_LT_WORKSPACE;
}

extern "C" int ptv3_pool_stage_fwd(const void* x, const void* weight, const void* bias, const float* coord,
                                   const int64_t* indices, const int64_t* idx_ptr, int64_t n, int64_t m, int c_in,
                                   int c_out, const float* bn_scale, const float* bn_shift, void* out,
                                   float* coord_out, int reduce, int dtype, void* workspace, size_t workspace_bytes,
                                   void* stream)
{
    PTV3_REQUIRE(dtype == PTV3_DTYPE_BF16 && c_in % 8 == 0 && c_out % 8 == 0 && c_in > 0 && c_out > 0,
                 PTV3_ERR_UNSUPPORTED, "ptv3_pool_stage_fwd: bf16 only, channel counts multiples of 8");
    PTV3_REQUIRE(n >= 0 && m >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_stage_fwd: bad sizes");
    if (n == 0 || m == 0) return PTV3_OK;
    PTV3_REQUIRE(x && weight && bias && indices && idx_ptr && out && workspace, PTV3_ERR_INVALID_ARGUMENT,
                 "ptv3_pool_stage_fwd: null pointer");
    PTV3_REQUIRE(workspace_bytes >= ptv3_pool_stage_workspace_bytes(n, c_out), PTV3_ERR_WORKSPACE,
                 "ptv3_pool_stage_fwd: workspace too small");
    Carver cv(workspace);
    char* proj = cv.take<char>((size_t)n * c_out * 2);
    char* lt = cv.take<char>(BLOCK_LT_WORKSPACE);
    int rc = gemm_bias_bf16(x, weight, bias, proj, n, c_in, c_out, lt, BLOCK_LT_WORKSPACE, (cudaStream_t)stream);
    if (rc != PTV3_OK) return rc;
    return ptv3_pool_fwd(proj, coord, indices, idx_ptr, m, c_out, bn_scale, bn_shift, out, coord_out, reduce, dtype,
                         stream);
}

extern "C" size_t ptv3_unpool_stage_workspace_bytes(int64_t n, int64_t m, int c_out)
{
    if (n <= 0 || m <= 0 || c_out <= 0) return 0;
    return align_up((size_t)n * c_out * 2, 256) + align_up((size_t)m * c_out * 2, 256) + BLOCK_LT_WORKSPACE;
}

extern "C" int ptv3_unpool_stage_fwd(const void* skip_feat, const void* child_feat, const void* w_skip,
                                     const void* b_skip, const void* w_child, const void* b_child,
                                     const int64_t* cluster, int64_t n, int64_t m, int c_skip, int c_child,
                                     int c_out, const float* skip_scale, const float* skip_shift,
                                     const float* child_scale, const float* child_shift, void* out,
                                     void* skip_act, int dtype, void* workspace, size_t workspace_bytes,
                                     void* stream)
{
    PTV3_REQUIRE(dtype == PTV3_DTYPE_BF16 && c_skip % 8 == 0 && c_child % 8 == 0 && c_out % 8 == 0 && c_skip > 0 &&
                     c_child > 0 && c_out > 0,
                 PTV3_ERR_UNSUPPORTED, "ptv3_unpool_stage_fwd: bf16 only, channel counts multiples of 8");
    PTV3_REQUIRE(n >= 0 && m >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_stage_fwd: bad sizes");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(m > 0 && skip_feat && child_feat && w_skip && b_skip && w_child && b_child && cluster && out &&
                     workspace,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_stage_fwd: null pointer or empty coarse level");
    PTV3_REQUIRE(workspace_bytes >= ptv3_unpool_stage_workspace_bytes(n, m, c_out), PTV3_ERR_WORKSPACE,
                 "ptv3_unpool_stage_fwd: workspace too small");
    Carver cv(workspace);
    char* skip_lin = cv.take<char>((size_t)n * c_out * 2);
    char* child_lin = cv.take<char>((size_t)m * c_out * 2);
    char* lt = cv.take<char>(BLOCK_LT_WORKSPACE);
    int rc = gemm_bias_bf16(child_feat, w_child, b_child, child_lin, m, c_child, c_out, lt, BLOCK_LT_WORKSPACE,
                            (cudaStream_t)stream);
    if (rc != PTV3_OK) return rc;
    rc = gemm_bias_bf16(skip_feat, w_skip, b_skip, skip_lin, n, c_skip, c_out, lt, BLOCK_LT_WORKSPACE,
                        (cudaStream_t)stream);
    if (rc != PTV3_OK) return rc;
    return ptv3_unpool_fwd(skip_lin, child_lin, cluster, n, c_out, skip_scale, skip_shift, child_scale, child_shift,
                           out, skip_act, dtype, stream);
}
