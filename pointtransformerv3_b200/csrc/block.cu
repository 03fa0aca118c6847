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
// Channel widths up to 128 take the Linear layers with the LayerNorm / residual glue in
// their epilogue (linear_tc05.cu) and, up to 64, the fused MLP; wider blocks take the
// streamed-weight tensor-core kernel (gemm_tc05.cu) and the fused row kernel for the glue.
#include "common.cuh"
#include "vec.cuh"

namespace ptv3 {

// out = [residual +] act(x W^T + b) by whichever of the two tensor-core Linear kernels covers
// the shape
static bool linear_any_supported(int k, int n_out, bool epilogue)
{
    if (ptv3_gemm_supported(k, n_out, PTV3_DTYPE_BF16)) return true;
    return !epilogue && ptv3_linear_supported(k, n_out, 0, PTV3_DTYPE_BF16);
}

static int linear_any(const void* x, const void* w, const void* bias, const void* residual, void* out, int64_t n,
                      int k, int n_out, int gelu, uint32_t* status, void* stream)
{
    if (ptv3_gemm_supported(k, n_out, PTV3_DTYPE_BF16))
        return ptv3_gemm_fwd(x, w, bias, residual, out, n, k, n_out, gelu, PTV3_DTYPE_BF16, status, stream);
    if (!gelu && !residual && ptv3_linear_supported(k, n_out, 0, PTV3_DTYPE_BF16))
        return ptv3_linear_fwd(x, w, bias, out, n, k, n_out, PTV3_DTYPE_BF16, status, stream);
    set_error("no tensor-core Linear kernel for %d -> %d channels", k, n_out);
    return PTV3_ERR_UNSUPPORTED;
}

struct BlockBuffers {
    void *x, *f1, *a, *qkv, *att, *f2, *hidden, *acc32;
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
    if (b) *b = t;
    return c.off;
}

}  // namespace ptv3

using namespace ptv3;

extern "C" int ptv3_block_supported(int channels, int heads, int hidden, int dtype)
{
    if (!(dtype == PTV3_DTYPE_BF16 && heads > 0 && channels % heads == 0 && channels % 16 == 0 &&
          hidden % 16 == 0 && channels >= 16 && hidden >= 16))
        return 0;
    const int C = channels;
    const bool tc_lin = ptv3_linear_supported(C, C, 1, dtype) && ptv3_linear_supported(C, 3 * C, 0, dtype);
    const bool wide_lin = linear_any_supported(C, C, false) && linear_any_supported(C, 3 * C, false);
    const bool mlp = ptv3_mlp_supported(C, hidden, dtype) ||
                     (linear_any_supported(C, hidden, true) && linear_any_supported(hidden, C, true));
    return (tc_lin || wide_lin) && mlp;
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
                                dt, 0, a->status, stream_));

    const bool tc_lin = ptv3_linear_supported(C, C, 1, dt) && ptv3_linear_supported(C, 3 * C, 0, dt);
    if (tc_lin) {
        STEP(ptv3_linear_ln_fwd(b.x, a->cpe_w, a->cpe_b, a->feat, a->cpe_ln_w, a->cpe_ln_b, a->cpe_ln_eps, b.f1,
                                a->n1_w, a->n1_b, a->n1_eps, b.a, n, C, dt, a->status, stream_));
        STEP(ptv3_linear_fwd(b.a, a->qkv_w, a->qkv_b, b.qkv, n, C, 3 * C, dt, a->status, stream_));
    } else {
        // streamed-weight Linear, then f1 = feat + LN_cpe(.), a = LN_1(f1) in the fused row kernel
        // (the qkv buffer is free here and serves as the Linear's output)
        STEP(linear_any(b.x, a->cpe_w, a->cpe_b, nullptr, b.qkv, n, C, C, 0, a->status, stream_));
        STEP(ptv3_add_layernorm_fwd(b.qkv, a->feat, a->cpe_ln_w, a->cpe_ln_b, a->cpe_ln_eps, b.f1, a->n1_w, a->n1_b,
                                    a->n1_eps, b.a, n, C, dt, stream_));
        STEP(linear_any(b.a, a->qkv_w, a->qkv_b, nullptr, b.qkv, n, C, 3 * C, 0, a->status, stream_));
    }
    STEP(ptv3_attention_fwd(b.qkv, a->order, a->pad, a->unpad, a->cu_seqlens, b.att, n, a->n_seq, a->max_seqlen, C,
                            a->heads, a->scale, dt, a->attention_algo, a->status, stream_));
    const bool fused_mlp = ptv3_mlp_supported(C, a->hidden, dt) != 0;
    if (tc_lin) {
        STEP(ptv3_linear_ln_fwd(b.att, a->proj_w, a->proj_b, b.f1, nullptr, nullptr, 0.f, b.f2, a->n2_w, a->n2_b,
                                a->n2_eps, b.a, n, C, dt, a->status, stream_));
    } else {
        STEP(linear_any(b.att, a->proj_w, a->proj_b, nullptr, b.qkv, n, C, C, 0, a->status, stream_));
        STEP(ptv3_add_layernorm_fwd(b.qkv, b.f1, nullptr, nullptr, 0.f, b.f2, a->n2_w, a->n2_b, a->n2_eps, b.a, n, C,
                                    dt, stream_));
    }
    if (fused_mlp) {
        STEP(ptv3_mlp_fwd(b.a, a->fc1_w, a->fc1_b, a->fc2_w, a->fc2_b, b.f2, a->out, n, C, a->hidden, dt, a->status,
                          stream_));
    } else {
        // hidden = GELU(fc1(b)), out = f2 + fc2(hidden): bias, activation and residual in the epilogues
        STEP(linear_any(b.a, a->fc1_w, a->fc1_b, nullptr, b.hidden, n, C, a->hidden, 1, a->status, stream_));
        STEP(linear_any(b.hidden, a->fc2_w, a->fc2_b, b.f2, a->out, n, a->hidden, C, 0, a->status, stream_));
    }
#undef STEP
    return PTV3_OK;
}

// ---------------------------------------------------------------------------
// Stage transitions in one call each: the projection(s) on the tensor-core Linear kernels
// followed by the pooling / unpooling kernel (model.py:684-689, 707-710 and model.py:726-735, 744-746).
// ---------------------------------------------------------------------------
extern "C" int ptv3_pool_stage_supported(int c_in, int c_out, int dtype)
{
    return dtype == PTV3_DTYPE_BF16 && c_in > 0 && c_out > 0 && linear_any_supported(c_in, c_out, false);
}

extern "C" size_t ptv3_pool_stage_workspace_bytes(int64_t n, int c_out)
{
    if (n <= 0 || c_out <= 0) return 0;
    return align_up((size_t)n * c_out * 2, 256);
}

extern "C" int ptv3_pool_stage_fwd(const void* x, const void* weight, const void* bias, const float* coord,
                                   const int64_t* indices, const int64_t* idx_ptr, int64_t n, int64_t m, int c_in,
                                   int c_out, const float* bn_scale, const float* bn_shift, void* out,
                                   float* coord_out, int reduce, int dtype, uint32_t* status, void* workspace,
                                   size_t workspace_bytes, void* stream)
{
    PTV3_REQUIRE(ptv3_pool_stage_supported(c_in, c_out, dtype), PTV3_ERR_UNSUPPORTED,
                 "ptv3_pool_stage_fwd: bf16 only, and a projection %d -> %d that one of the tensor-core Linear "
                 "kernels takes", c_in, c_out);
    PTV3_REQUIRE(n >= 0 && m >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_stage_fwd: bad sizes");
    if (n == 0 || m == 0) return PTV3_OK;
    PTV3_REQUIRE(x && weight && bias && indices && idx_ptr && out && workspace && status,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_pool_stage_fwd: null pointer");
    PTV3_REQUIRE(workspace_bytes >= ptv3_pool_stage_workspace_bytes(n, c_out), PTV3_ERR_WORKSPACE,
                 "ptv3_pool_stage_fwd: workspace too small");
    Carver cv(workspace);
    char* proj = cv.take<char>((size_t)n * c_out * 2);
    int rc = linear_any(x, weight, bias, nullptr, proj, n, c_in, c_out, 0, status, stream);
    if (rc != PTV3_OK) return rc;
    return ptv3_pool_fwd(proj, coord, indices, idx_ptr, m, c_out, bn_scale, bn_shift, out, coord_out, reduce, dtype,
                         stream);
}

extern "C" size_t ptv3_unpool_stage_workspace_bytes(int64_t n, int64_t m, int c_out)
{
    if (n <= 0 || m <= 0 || c_out <= 0) return 0;
    return align_up((size_t)n * c_out * 2, 256) + align_up((size_t)m * c_out * 2, 256);
}

extern "C" int ptv3_unpool_stage_fwd(const void* skip_feat, const void* child_feat, const void* w_skip,
                                     const void* b_skip, const void* w_child, const void* b_child,
                                     const int64_t* cluster, int64_t n, int64_t m, int c_skip, int c_child,
                                     int c_out, const float* skip_scale, const float* skip_shift,
                                     const float* child_scale, const float* child_shift, void* out,
                                     void* skip_act, int dtype, uint32_t* status, void* workspace,
                                     size_t workspace_bytes, void* stream)
{
    PTV3_REQUIRE(ptv3_pool_stage_supported(c_skip, c_out, dtype) && ptv3_pool_stage_supported(c_child, c_out, dtype),
                 PTV3_ERR_UNSUPPORTED,
                 "ptv3_unpool_stage_fwd: bf16 only, and projections %d -> %d, %d -> %d that the tensor-core Linear "
                 "kernels take", c_skip, c_out, c_child, c_out);
    PTV3_REQUIRE(n >= 0 && m >= 0, PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_stage_fwd: bad sizes");
    if (n == 0) return PTV3_OK;
    PTV3_REQUIRE(m > 0 && skip_feat && child_feat && w_skip && b_skip && w_child && b_child && cluster && out &&
                     workspace && status,
                 PTV3_ERR_INVALID_ARGUMENT, "ptv3_unpool_stage_fwd: null pointer or empty coarse level");
    PTV3_REQUIRE(workspace_bytes >= ptv3_unpool_stage_workspace_bytes(n, m, c_out), PTV3_ERR_WORKSPACE,
                 "ptv3_unpool_stage_fwd: workspace too small");
    Carver cv(workspace);
    char* skip_lin = cv.take<char>((size_t)n * c_out * 2);
    char* child_lin = cv.take<char>((size_t)m * c_out * 2);
    int rc = linear_any(child_feat, w_child, b_child, nullptr, child_lin, m, c_child, c_out, 0, status, stream);
    if (rc != PTV3_OK) return rc;
    rc = linear_any(skip_feat, w_skip, b_skip, nullptr, skip_lin, n, c_skip, c_out, 0, status, stream);
    if (rc != PTV3_OK) return rc;
    return ptv3_unpool_fwd(skip_lin, child_lin, cluster, n, c_out, skip_scale, skip_shift, child_scale, child_shift,
                           out, skip_act, dtype, stream);
}
