"""ctypes binding of libptv3_b200.so (the C ABI declared in include/ptv3_b200.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised."""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libptv3_b200.so")

c_i64 = ctypes.c_int64
c_int = ctypes.c_int
c_f32 = ctypes.c_float
c_sz = ctypes.c_size_t
c_ptr = ctypes.c_void_p



class BlockArgs(ctypes.Structure):
    """ptv3_block_args of include/ptv3_b200.h (same field order)."""
    _fields_ = (
        [("n", c_i64), ("channels", c_int), ("heads", c_int), ("hidden", c_int), ("dtype", c_int),
         ("n_seq", c_int), ("max_seqlen", c_int), ("attention_algo", c_int), ("scale", c_f32),
         ("cpe_ln_eps", c_f32), ("n1_eps", c_f32), ("n2_eps", c_f32)]
        + [(name, c_ptr) for name in (
            "conv_in", "feat", "out", "nbr", "row_order", "pair_in", "pair_out", "off_start", "tile_start",
            "order", "pad", "unpad", "cu_seqlens", "conv_weight", "conv_bias", "cpe_w", "cpe_b", "cpe_ln_w",
            "cpe_ln_b", "n1_w", "n1_b", "qkv_w", "qkv_b", "proj_w", "proj_b", "n2_w", "n2_b", "fc1_w", "fc1_b",
            "fc2_w", "fc2_b", "status", "workspace")]
        + [("workspace_bytes", c_sz)])


# name -> (restype, argtypes); must list every symbol of include/ptv3_b200.h
SIGNATURES = {
    "ptv3_last_error": (ctypes.c_char_p, []),
    "ptv3_version": (c_int, []),
    "ptv3_launch_count": (ctypes.c_longlong, []),
    "ptv3_encode": (c_int, [c_ptr, c_ptr, c_i64, c_int, ctypes.POINTER(c_int), c_int, c_ptr, c_ptr]),
    "ptv3_decode": (c_int, [c_ptr, c_i64, c_int, c_int, c_ptr, c_ptr, c_ptr]),
    "ptv3_argsort_workspace_bytes": (c_sz, [c_int, c_i64, c_int]),
    "ptv3_argsort_inverse": (c_int, [c_ptr, c_int, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_pad_plan": (c_int, [c_ptr, c_int, c_int, c_i64, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr]),
    "ptv3_attention_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int,
                                   c_int, c_f32, c_int, c_int, c_ptr, c_ptr]),
    "ptv3_attention_rpe_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_i64, c_int,
                                       c_int, c_int, c_int, c_f32, c_int, c_ptr]),
    "ptv3_kmap_workspace_bytes": (c_sz, [c_i64]),
    "ptv3_status_reset": (c_int, [c_ptr, c_ptr]),
    "ptv3_batch_indices": (c_int, [c_ptr, c_int, c_ptr, c_i64, c_ptr, c_ptr, c_ptr]),
    "ptv3_kmap_build": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_kmap_build_ordered": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_kmap_static_max_voxels": (c_i64, []),
    "ptv3_kmap_build_static": (c_int, [c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr]),
    "ptv3_subm_conv_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int,
                                   c_int, c_int, c_ptr, c_ptr]),
    "ptv3_conv_pairs_workspace_bytes": (c_sz, [c_i64, c_int]),
    "ptv3_conv_pairs_build": (c_int, [c_ptr, c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_subm_conv_pairs_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_sz,
                                         c_i64, c_int, c_int, c_int, c_int, c_ptr]),
    "ptv3_subm_conv_direct_workspace_bytes": (c_sz, [c_i64, c_int]),
    "ptv3_subm_conv_direct_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_i64,
                                          c_int, c_int, c_int, c_int, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_pool_plan_workspace_bytes": (c_sz, [c_int, c_i64, c_int]),
    "ptv3_pool_plan": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_i64, c_int, c_int,
                               ctypes.POINTER(c_int), c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                               c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_pool_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_int,
                              c_ptr]),
    "ptv3_add_layernorm_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_f32, c_ptr,
                                       c_i64, c_int, c_int, c_ptr]),
    "ptv3_linear_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "ptv3_gemm_supported": (c_int, [c_int, c_int, c_int]),
    "ptv3_gemm_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int, c_int, c_ptr, c_ptr]),
    "ptv3_linear_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int, c_ptr, c_ptr]),
    "ptv3_linear_ln_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_f32, c_ptr, c_ptr, c_ptr, c_f32,
                                   c_ptr, c_i64, c_int, c_int, c_ptr, c_ptr]),
    "ptv3_mlp_supported": (c_int, [c_int, c_int, c_int]),
    "ptv3_mlp_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int, c_ptr,
                             c_ptr]),
    "ptv3_grid_coord": (c_int, [c_ptr, c_i64, c_f32, c_ptr, c_ptr, c_ptr]),
    "ptv3_voxel_dedup_workspace_bytes": (c_sz, [c_i64]),
    "ptv3_voxel_dedup": (c_int, [c_ptr, c_i64, c_ptr, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_seg_head_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_int, c_int, c_int, c_ptr]),
    "ptv3_pool_stage_supported": (c_int, [c_int, c_int, c_int]),
    "ptv3_pool_stage_workspace_bytes": (c_sz, [c_i64, c_int]),
    "ptv3_pool_stage_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_int, c_int, c_ptr, c_ptr,
                                    c_ptr, c_ptr, c_int, c_int, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_unpool_stage_workspace_bytes": (c_sz, [c_i64, c_i64, c_int]),
    "ptv3_unpool_stage_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_i64, c_i64, c_int, c_int,
                                      c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr, c_int, c_ptr, c_ptr, c_sz, c_ptr]),
    "ptv3_block_supported": (c_int, [c_int, c_int, c_int, c_int]),
    "ptv3_block_workspace_bytes": (c_sz, [ctypes.POINTER(BlockArgs)]),
    "ptv3_block_fwd": (c_int, [ctypes.POINTER(BlockArgs), c_ptr]),
    "ptv3_unpool_fwd": (c_int, [c_ptr, c_ptr, c_ptr, c_i64, c_int, c_ptr, c_ptr, c_ptr, c_ptr, c_ptr,
                                c_ptr, c_int, c_ptr]),
}

_lib = None


class Ptv3Error(RuntimeError):
    pass


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise Ptv3Error(
                "CUDA library %s is not built; run `python -m pointtransformerv3_b200.build` "
                "(there is no CPU fallback)" % LIB_PATH)
        lib = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc, what):
    if rc != 0:
        raise Ptv3Error("%s failed (%d): %s" % (what, rc, load().ptv3_last_error().decode()))


def ptr(t):
    """Device pointer of a tensor (None -> NULL)."""
    if t is None:
        return None
    return t.data_ptr()


def stream():
    """Raw handle of the current CUDA stream of the current device (the private
    torch accessor is an order of magnitude cheaper than building a Stream
    object on every operator call)."""
    try:
        return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())
    except AttributeError:
        return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise Ptv3Error("tensor on %s: this library has CUDA kernels only, no CPU path" % t.device)


def workspace(nbytes, device):
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


DTYPE_IDS = {torch.float32: 0, torch.bfloat16: 1}


def dtype_id(t):
    try:
        return DTYPE_IDS[t.dtype]
    except KeyError:
        raise Ptv3Error("feature dtype %s is not supported (float32 or bfloat16)" % t.dtype)


STATUS_BITS = {1: "index or size out of range", 2: "hash probe limit reached", 4: "device wait limit reached"}


def raise_on_status(status, what):
    """Reads the device status word (one host sync) and raises if a bit is set."""
    v = int(status.item())
    if v:
        msg = ", ".join(m for b, m in STATUS_BITS.items() if v & b)
        raise Ptv3Error("%s: device status 0x%x (%s)" % (what, v, msg))
