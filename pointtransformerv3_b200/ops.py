"""Thin tensor-level wrappers over the C ABI (one function per entry point).

Every wrapper allocates outputs and workspaces with torch, passes raw device
pointers and the current CUDA stream, and raises on a non-zero status."""
import ctypes
import threading
import time

import torch

from . import _lib

ORDER_IDS = {"z": 0, "z-trans": 1, "hilbert": 2, "hilbert-trans": 3}

# Optional per-operator device timing: when TIMERS is a dict, every wrapped call
# records a CUDA event pair on the current stream under the operator's name,
# together with the `work` figure (algorithmic FLOPs or bytes) of the call.
TIMERS = None
TIMER_FILTER = None     # optional set of operator names to time (None = all)


class timed:
    def __init__(self, name, work=0.0, extra=0.0):
        self.name, self.work, self.extra = name, work, extra

    def __enter__(self):
        self.on = TIMERS is not None and (TIMER_FILTER is None or self.name in TIMER_FILTER)
        if self.on:
            self.start = torch.cuda.Event(enable_timing=True)
            self.end = torch.cuda.Event(enable_timing=True)
            self.start.record()
        return self

    def __exit__(self, *exc):
        if self.on:
            self.end.record()
            TIMERS.setdefault(self.name, []).append((self.start, self.end, self.work, self.extra))
        return False


def timer_summary():
    """name -> dict(calls, ms, work, extra) from the recorded events (synchronises)."""
    torch.cuda.synchronize()
    out = {}
    for name, evs in (TIMERS or {}).items():
        out[name] = dict(calls=len(evs), ms=sum(e[0].elapsed_time(e[1]) for e in evs),
                         work=sum(e[2] for e in evs), extra=sum(e[3] for e in evs))
    return out


def encode(grid_coord, batch, depth, orders):
    """grid_coord (N,3) integer CUDA tensor, batch (N,) or None, orders: list of
    names -> (len(orders), N) int64 codes."""
    _lib.require_cuda(grid_coord, batch)
    lib = _lib.load()
    if grid_coord.dim() != 2 or grid_coord.shape[1] != 3:
        raise ValueError("grid_coord must be (N, 3), got %s" % (tuple(grid_coord.shape),))
    g = grid_coord.to(torch.int32).contiguous()
    n = g.shape[0]
    b = None
    if batch is not None:
        b = batch.to(torch.int64).contiguous()
        if b.shape != (n,):
            raise ValueError("batch must be (N,)")
    ids = (ctypes.c_int * len(orders))(*[ORDER_IDS[o] for o in orders])
    codes = torch.empty((len(orders), n), dtype=torch.int64, device=g.device)
    with timed("encode", n * (12.0 + (8.0 if b is not None else 0.0) + 8.0 * len(orders))):
        _lib.check(lib.ptv3_encode(_lib.ptr(g), _lib.ptr(b), n, int(depth), ids, len(orders),
                                   _lib.ptr(codes), _lib.stream()), "ptv3_encode")
    return codes


def decode(code, depth, order):
    """(N,) int64 codes -> (grid_coord (N,3) int64, batch (N,) int64); order "z" or "hilbert"."""
    _lib.require_cuda(code)
    lib = _lib.load()
    code = code.to(torch.int64).contiguous().reshape(-1)
    n = code.shape[0]
    grid = torch.empty((n, 3), dtype=torch.int64, device=code.device)
    batch = torch.empty(n, dtype=torch.int64, device=code.device)
    _lib.check(lib.ptv3_decode(_lib.ptr(code), n, int(depth), ORDER_IDS[order], _lib.ptr(grid), _lib.ptr(batch),
                               _lib.stream()), "ptv3_decode")
    return grid, batch


def argsort_inverse(codes, sig_bits, status=None):
    """codes (k,N) int64 -> (order, inverse), both (k,N) int64, stable.  status: the
    caller's device status word (checked by the caller); without one a private word is
    made and checked here."""
    _lib.require_cuda(codes)
    lib = _lib.load()
    codes = codes.contiguous()
    k, n = codes.shape
    order = torch.empty_like(codes)
    inverse = torch.empty_like(codes)
    nbytes = lib.ptv3_argsort_workspace_bytes(k, n, int(sig_bits))
    ws = _lib.workspace(nbytes, codes.device)
    own = status is None
    if own:
        status = new_status(codes.device)
    with timed("argsort_inverse", 24.0 * k * n):
        _lib.check(lib.ptv3_argsort_inverse(_lib.ptr(codes), k, n, int(sig_bits), _lib.ptr(order),
                                            _lib.ptr(inverse), _lib.ptr(status), _lib.ptr(ws), nbytes,
                                            _lib.stream()),
                   "ptv3_argsort_inverse")
    if own:
        _lib.raise_on_status(status, "ptv3_argsort_inverse")
    return order, inverse


def new_status(device):
    """A cleared device status word (cleared by a memset in stream order)."""
    device = torch.device(device)
    if device.type != "cuda":
        return torch.zeros(1, dtype=torch.int32, device=device)
    status = torch.empty(1, dtype=torch.int32, device=device)
    _lib.check(_lib.load().ptv3_status_reset(_lib.ptr(status), _lib.stream()), "ptv3_status_reset")
    return status


def pad_layout(counts, patch):
    """Host arithmetic of model.py:392-404: (n_pad, n_seq) from per-scene counts."""
    n_pad = n_seq = 0
    for c in counts:
        cp = (c + patch - 1) // patch * patch if c > patch else c
        n_pad += cp
        n_seq += (cp + patch - 1) // patch
    return n_pad, n_seq


def pad_plan(offset, counts, patch, status=None):
    """offset (B,) int64 CUDA, counts: the same as host ints -> (pad, unpad, cu_seqlens)."""
    _lib.require_cuda(offset)
    lib = _lib.load()
    offset = offset.to(torch.int64).contiguous()
    n = int(sum(counts))
    n_pad, n_seq = pad_layout(counts, patch)
    dev = offset.device
    pad = torch.empty(n_pad, dtype=torch.int64, device=dev)
    unpad = torch.empty(n, dtype=torch.int64, device=dev)
    cu = torch.empty(n_seq + 1, dtype=torch.int32, device=dev)
    own = status is None
    if own:
        status = new_status(dev)
    _lib.check(lib.ptv3_pad_plan(_lib.ptr(offset), len(counts), int(patch), n, n_pad, n_seq,
                                 _lib.ptr(pad), _lib.ptr(unpad), _lib.ptr(cu), _lib.ptr(status),
                                 _lib.stream()), "ptv3_pad_plan")
    if own:
        _lib.raise_on_status(status, "ptv3_pad_plan")
    return pad, unpad, cu


def attention(qkv, order_row, pad, unpad, cu_seqlens, heads, max_seqlen, scale, algo=0, status=None):
    """qkv (N, 3C) -> (N, C): the attention core between the two Linear layers.
    status: the caller's device status word (checked by the caller); without
    one a private word is made and checked here."""
    _lib.require_cuda(qkv, order_row, pad, unpad, cu_seqlens)
    lib = _lib.load()
    qkv = qkv.contiguous()
    n, c3 = qkv.shape
    C = c3 // 3
    out = torch.empty((n, C), dtype=qkv.dtype, device=qkv.device)
    own = status is None
    if own:
        status = new_status(qkv.device)
    # algorithmic work: QK^T and PV of every sequence, 4 L^2 C FLOPs (read from the device only
    # while per-operator timing is on)
    work = 0.0
    if TIMERS is not None:
        work = 4.0 * C * float(torch.diff(cu_seqlens).double().square().sum().item())
    with timed("attention", work, float(pad.numel()) * C):      # extra: padded rows x channels
        _lib.check(lib.ptv3_attention_fwd(_lib.ptr(qkv), _lib.ptr(order_row.contiguous()), _lib.ptr(pad),
                                          _lib.ptr(unpad), _lib.ptr(cu_seqlens), _lib.ptr(out), n,
                                          cu_seqlens.numel() - 1, int(max_seqlen), C, int(heads),
                                          float(scale), _lib.dtype_id(qkv), int(algo), _lib.ptr(status),
                                          _lib.stream()),
                   "ptv3_attention_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_attention_fwd")
    return out


def attention_rpe(qkv, order_row, pad, unpad, cu_seqlens, grid_coord, rpe_table, pos_bnd, heads, max_seqlen,
                  scale):
    """Patch attention with the relative position bias (see ptv3_attention_rpe_fwd)."""
    _lib.require_cuda(qkv, order_row, pad, unpad, cu_seqlens, grid_coord, rpe_table)
    lib = _lib.load()
    qkv = qkv.contiguous()
    n, c3 = qkv.shape
    C = c3 // 3
    grid_coord = grid_coord.to(torch.int32).contiguous()
    rpe_table = rpe_table.to(torch.float32).contiguous()
    out = torch.empty((n, C), dtype=qkv.dtype, device=qkv.device)
    with timed("attention_rpe", 4.0 * pad.numel() * max_seqlen * C):
        _lib.check(lib.ptv3_attention_rpe_fwd(_lib.ptr(qkv), _lib.ptr(order_row.contiguous()), _lib.ptr(pad),
                                              _lib.ptr(unpad), _lib.ptr(cu_seqlens), _lib.ptr(grid_coord),
                                              _lib.ptr(rpe_table), int(pos_bnd), _lib.ptr(out), n,
                                              cu_seqlens.numel() - 1, int(max_seqlen), C, int(heads), float(scale),
                                              _lib.dtype_id(qkv), _lib.stream()), "ptv3_attention_rpe_fwd")
    return out


def batch_indices(offset, n, grid_coord=None, want_batch=True):
    """(batch, indices): the scene index of each of the n points (int64) and, with grid_coord, the
    (n, 4) int32 rows (batch, x, y, z) of the sparse tensor; one kernel, no device read."""
    _lib.require_cuda(offset, grid_coord)
    lib = _lib.load()
    offset = offset.to(torch.int64).contiguous()
    n = int(n)
    dev = offset.device
    batch = torch.empty(n, dtype=torch.int64, device=dev) if want_batch else None
    indices = None
    if grid_coord is not None:
        grid_coord = grid_coord.to(torch.int32).contiguous()
        if grid_coord.shape != (n, 3):
            raise ValueError("grid_coord must be (n, 3)")
        indices = torch.empty((n, 4), dtype=torch.int32, device=dev)
    _lib.check(lib.ptv3_batch_indices(_lib.ptr(offset), offset.shape[0], _lib.ptr(grid_coord), n, _lib.ptr(batch),
                                      _lib.ptr(indices), _lib.stream()), "ptv3_batch_indices")
    return batch, indices


def kmap_build(indices, ksize, status=None, row_order=None):
    """indices (N,4) int32 (b,x,y,z) -> nbr (ksize^3, N) int32, offset-major.
    row_order: optional (N,) int64 permutation; column p then describes voxel row_order[p]
    (the table of the natural order with its columns permuted)."""
    _lib.require_cuda(indices, row_order)
    lib = _lib.load()
    indices = indices.to(torch.int32).contiguous()
    n = indices.shape[0]
    nbr = torch.empty((ksize ** 3, n), dtype=torch.int32, device=indices.device)
    nbytes = lib.ptv3_kmap_workspace_bytes(n)
    ws = _lib.workspace(nbytes, indices.device)
    own = status is None
    if own:
        status = new_status(indices.device)
    with timed("kmap_k%d" % ksize, n * (16.0 + 4.0 * ksize ** 3)):
        if row_order is not None:
            row_order = row_order.to(torch.int64).contiguous()
            if row_order.shape != (n,):
                raise ValueError("row_order must hold one entry per voxel")
        _lib.check(lib.ptv3_kmap_build_ordered(_lib.ptr(indices), n, int(ksize), _lib.ptr(row_order), _lib.ptr(nbr),
                                               _lib.ptr(status), _lib.ptr(ws), nbytes, _lib.stream()),
                   "ptv3_kmap_build")
    if own:
        _lib.raise_on_status(status, "ptv3_kmap_build")
    return nbr


def subm_conv(feat, nbr, weight, bias=None, algo=0, row_order=None, status=None):
    """feat (N,Cin), nbr (k^3,N) int32, weight (Cout,k,k,k,Cin) -> (N,Cout).
    row_order: optional (N,) int64 permutation used to group voxels into tiles.
    status: device status word of the caller (read later); without one a fresh word
    is made and checked here (one host sync)."""
    _lib.require_cuda(feat, nbr, weight, bias)
    lib = _lib.load()
    feat = feat.contiguous()
    n, cin = feat.shape
    cout = weight.shape[0]
    kvol = nbr.shape[0]
    if weight.numel() != cout * kvol * cin or weight.dtype != feat.dtype:
        raise ValueError("weight %s/%s does not match feat %s/%s and %d offsets" % (
            tuple(weight.shape), weight.dtype, tuple(feat.shape), feat.dtype, kvol))
    if bias is not None and bias.dtype != feat.dtype:
        raise ValueError("bias dtype %s != feature dtype %s" % (bias.dtype, feat.dtype))
    out = torch.empty((n, cout), dtype=feat.dtype, device=feat.device)
    own = status is None
    if own:
        status = new_status(feat.device)
    with timed("subm_conv_k%d" % round(kvol ** (1 / 3)), 2.0 * n * kvol * cin * cout):
        _lib.check(lib.ptv3_subm_conv_fwd(_lib.ptr(feat), _lib.ptr(nbr), _lib.ptr(weight.contiguous()),
                                          _lib.ptr(bias), _lib.ptr(out), _lib.ptr(row_order), n, cin, cout, kvol,
                                          _lib.dtype_id(feat), int(algo), _lib.ptr(status), _lib.stream()),
                   "ptv3_subm_conv_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_subm_conv_fwd")
    return out


def _offsets_to_device(counts, dev):
    """Cumulative counts as a device tensor: summed on the host (the counts are there already) and
    copied from pinned memory in stream order.  The pinned words are reused by the next plan, which
    the host only starts after it has waited for kernels queued behind this copy."""
    off_host = _pinned(len(counts), torch.int64, "pool_plan.offset")
    acc = 0
    for i, c in enumerate(counts):
        acc += int(c)
        off_host[i] = acc
    return off_host.to(dev, non_blocking=True)


def pool_plan(code, order, grid_coord, batch, n_scenes, pooling_depth, row_perm=None, status=None):
    """Builds the pooled level's index tensors; one host sync to learn its size.

    Returns dict(cluster, idx_ptr, head, code, order, inverse, grid_coord, batch, counts,
    offset, m)."""
    _lib.require_cuda(code, order, grid_coord, batch)
    lib = _lib.load()
    code, order = code.contiguous(), order.contiguous()
    grid_coord = grid_coord.to(torch.int32).contiguous()
    batch = batch.to(torch.int64).contiguous()
    k, n = code.shape
    dev = code.device
    i64 = dict(dtype=torch.int64, device=dev)
    cluster = torch.empty(n, **i64)
    idx_ptr = torch.empty(n + 1, **i64)
    head = torch.empty(n, **i64)
    pcode = torch.empty((k, n), **i64)
    porder = torch.empty((k, n), **i64)
    pinv = torch.empty((k, n), **i64)
    pgrid = torch.empty((n, 3), dtype=torch.int32, device=dev)
    pbatch = torch.empty(n, **i64)
    meta = torch.empty(1 + n_scenes, **i64)
    if status is None:
        status = new_status(dev)
    nbytes = lib.ptv3_pool_plan_workspace_bytes(k, n, n_scenes)
    ws = _lib.workspace(nbytes, dev)
    perm = None
    if row_perm is not None:
        perm = (ctypes.c_int * k)(*[int(v) for v in row_perm])
    # the sizes of the coarse level and the status word arrive in mapped host memory, written by
    # the plan's last kernel; the host polls the "done" word behind them (a stream wait through
    # the driver takes several times longer to notice the end of a kernel)
    meta_host = _pinned(3 + n_scenes, torch.int64, "pool_plan.meta")
    meta_host[-1] = 0
    _lib.check(lib.ptv3_pool_plan(_lib.ptr(code), _lib.ptr(order), _lib.ptr(grid_coord), _lib.ptr(batch),
                                  k, n, n_scenes, int(pooling_depth), perm, _lib.ptr(cluster),
                                  _lib.ptr(idx_ptr), _lib.ptr(head), _lib.ptr(pcode), _lib.ptr(porder),
                                  _lib.ptr(pinv), _lib.ptr(pgrid), _lib.ptr(pbatch), _lib.ptr(meta),
                                  ctypes.c_void_p(meta_host.data_ptr()), _lib.ptr(status), _lib.ptr(ws), nbytes,
                                  _lib.stream()),
               "ptv3_pool_plan")
    _wait_flag(meta_host)                          # the one wait
    host = meta_host.tolist()[:-1]
    if host[-1]:
        raise _lib.Ptv3Error("device status 0x%x (read after ptv3_pool_plan; the word is shared by "
                             "every kernel queued with it)" % host[-1])
    host = host[:-1]
    m = host[0]
    # the k-row outputs are written packed (row stride m): views, no copies
    packed = lambda t: t.view(-1)[: k * m].view(k, m)
    return dict(cluster=cluster, idx_ptr=idx_ptr[: m + 1], head=head[:m],
                code=packed(pcode), order=packed(porder), inverse=packed(pinv), grid_coord=pgrid[:m],
                batch=pbatch[:m], counts=host[1:], m=m, offset=_offsets_to_device(host[1:], dev))


POLL_SECONDS = 2.0      # how long a host thread polls a "done" word before it asks the driver


def _wait_flag(buf):
    """Waits until the last word of the pinned tensor ``buf`` is non-zero (stored by the last
    kernel of a call).  Falls back to waiting for the stream, so a failed launch cannot hang
    the host."""
    flag = buf[-1:]
    deadline = None
    while int(flag) == 0:
        if deadline is None:
            deadline = time.monotonic() + POLL_SECONDS
        elif time.monotonic() > deadline:
            torch.cuda.current_stream().synchronize()
            if int(flag) == 0:
                raise _lib.Ptv3Error("the kernels of this call finished without reporting their result")
            break


_PINNED = {}


def _pinned(numel, dtype, tag):
    """A cached pinned host buffer per call site, host thread and CUDA stream (a caller
    synchronises its stream before reading the buffer, so calls that share all three do
    not overlap)."""
    key = (tag, numel, dtype, threading.get_ident(), torch.cuda.current_stream().cuda_stream)
    buf = _PINNED.get(key)
    if buf is None:
        with torch.inference_mode(False):      # a plain tensor: it is written in and out of inference mode
            buf = torch.empty(numel, dtype=dtype).pin_memory()
        _PINNED[key] = buf
    return buf


REDUCE_IDS = {"max": 0, "min": 1, "sum": 2, "mean": 3}


def pool(x, coord, indices, idx_ptr, bn_scale=None, bn_shift=None, reduce="max"):
    """Segment reduction (+ BN + GELU) of x and mean of coord over clusters."""
    _lib.require_cuda(x, indices, idx_ptr)
    lib = _lib.load()
    x = x.contiguous()
    m = idx_ptr.numel() - 1
    C = x.shape[1]
    out = torch.empty((m, C), dtype=x.dtype, device=x.device)
    cout = None
    if coord is not None:
        coord = coord.to(torch.float32).contiguous()
        cout = torch.empty((m, 3), dtype=torch.float32, device=x.device)
    _lib.check(lib.ptv3_pool_fwd(_lib.ptr(x), _lib.ptr(coord), _lib.ptr(indices), _lib.ptr(idx_ptr), m, C,
                                 _lib.ptr(bn_scale), _lib.ptr(bn_shift), _lib.ptr(out), _lib.ptr(cout),
                                 REDUCE_IDS[reduce], _lib.dtype_id(x), _lib.stream()), "ptv3_pool_fwd")
    return out, cout


def unpool(skip, child, cluster, skip_scale, skip_shift, child_scale, child_shift, want_skip_act=True):
    _lib.require_cuda(skip, child, cluster)
    lib = _lib.load()
    skip, child = skip.contiguous(), child.contiguous()
    n, C = skip.shape
    out = torch.empty_like(skip)
    act = torch.empty_like(skip) if want_skip_act else None
    _lib.check(lib.ptv3_unpool_fwd(_lib.ptr(skip), _lib.ptr(child), _lib.ptr(cluster), n, C,
                                   _lib.ptr(skip_scale), _lib.ptr(skip_shift), _lib.ptr(child_scale),
                                   _lib.ptr(child_shift), _lib.ptr(out), _lib.ptr(act),
                                   _lib.dtype_id(skip), _lib.stream()), "ptv3_unpool_fwd")
    return out, act


def add_layernorm(x, residual=None, ln1=None, ln2=None, want_sum=True):
    """Fused glue of a block: t = LN1(x) (or x), s = residual + t (or t),
    y = LN2(s).  ln1/ln2 are torch.nn.LayerNorm modules or None.
    Returns (s or None, y or None)."""
    _lib.require_cuda(x, residual)
    lib = _lib.load()
    x = x.contiguous()
    n, C = x.shape
    if residual is not None:
        residual = residual.contiguous()
        if residual.shape != x.shape or residual.dtype != x.dtype:
            raise ValueError("residual must match x")

    def params(ln):
        if ln is None:
            return None, None, 0.0
        if ln.weight is None or ln.bias is None or tuple(ln.normalized_shape) != (C,):
            raise ValueError("LayerNorm must be affine over the channel axis")
        if ln.weight.dtype != x.dtype:
            raise ValueError("LayerNorm parameters must have the feature dtype")
        return ln.weight, ln.bias, float(ln.eps)
    w1, b1, e1 = params(ln1)
    w2, b2, e2 = params(ln2)
    s = torch.empty_like(x) if (want_sum or ln2 is None) else None
    y = torch.empty_like(x) if ln2 is not None else None
    with timed("add_layernorm", float(x.numel() * x.element_size()) * (1 + (residual is not None) +
                                                                       (s is not None) + (y is not None))):
        _lib.check(lib.ptv3_add_layernorm_fwd(_lib.ptr(x), _lib.ptr(residual), _lib.ptr(w1), _lib.ptr(b1), e1,
                                              _lib.ptr(s), _lib.ptr(w2), _lib.ptr(b2), e2, _lib.ptr(y), n, C,
                                              _lib.dtype_id(x), _lib.stream()), "ptv3_add_layernorm_fwd")
    return s, y


def subm_conv_direct(feat, indices, weight, bias=None, bn_scale=None, bn_shift=None, gelu=False,
                     row_order=None, status=None):
    """Submanifold convolution for few input channels / large kernels that probes
    the voxel hash table itself (no kernel map); optional fused BN(eval) + GELU."""
    _lib.require_cuda(feat, indices, weight, bias)
    lib = _lib.load()
    feat = feat.contiguous()
    indices = indices.to(torch.int32).contiguous()
    n, cin = feat.shape
    cout, ksize = weight.shape[0], weight.shape[1]
    if weight.dtype != feat.dtype or weight.shape[-1] != cin:
        raise ValueError("weight does not match the features")
    out = torch.empty((n, cout), dtype=feat.dtype, device=feat.device)
    nbytes = lib.ptv3_subm_conv_direct_workspace_bytes(n, ksize)
    ws = _lib.workspace(nbytes, feat.device)
    own = status is None
    if own:
        status = new_status(feat.device)
    with timed("subm_conv_direct_k%d" % ksize, 2.0 * n * ksize ** 3 * cin * cout):
        _lib.check(lib.ptv3_subm_conv_direct_fwd(
            _lib.ptr(feat), _lib.ptr(indices), _lib.ptr(weight.contiguous()), _lib.ptr(bias),
            _lib.ptr(bn_scale), _lib.ptr(bn_shift), int(bool(gelu)), _lib.ptr(out), _lib.ptr(row_order), n, cin,
            cout, ksize, _lib.dtype_id(feat), _lib.ptr(status), _lib.ptr(ws), nbytes, _lib.stream()),
            "ptv3_subm_conv_direct_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_subm_conv_direct_fwd")
    return out


def mlp_supported(channels, hidden, dtype):
    return dtype in _lib.DTYPE_IDS and bool(_lib.load().ptv3_mlp_supported(channels, hidden, _lib.DTYPE_IDS[dtype]))


def mlp(x, fc1_weight, fc1_bias, fc2_weight, fc2_bias, residual, status=None):
    """out = residual + fc2(GELU(fc1(x))) in one kernel (see ptv3_mlp_fwd)."""
    _lib.require_cuda(x, fc1_weight, fc2_weight, residual)
    lib = _lib.load()
    x, residual = x.contiguous(), residual.contiguous()
    n, C = x.shape
    hidden = fc1_weight.shape[0]
    out = torch.empty_like(x)
    own = status is None
    if own:
        status = new_status(x.device)
    with timed("mlp", 4.0 * n * C * hidden):
        _lib.check(lib.ptv3_mlp_fwd(_lib.ptr(x), _lib.ptr(fc1_weight.contiguous()), _lib.ptr(fc1_bias),
                                    _lib.ptr(fc2_weight.contiguous()), _lib.ptr(fc2_bias), _lib.ptr(residual),
                                    _lib.ptr(out), n, C, hidden, _lib.dtype_id(x), _lib.ptr(status),
                                    _lib.stream()), "ptv3_mlp_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_mlp_fwd")
    return out


def conv_pairs_build(nbr, row_order=None):
    """Offset-sorted (input row, output row) pair list of a neighbour table.
    Returns dict(pair_in, pair_out, off_start, tile_start) of device tensors."""
    _lib.require_cuda(nbr, row_order)
    lib = _lib.load()
    kvol, n = nbr.shape
    dev = nbr.device
    i32 = dict(dtype=torch.int32, device=dev)
    pair_in = torch.empty(kvol * n, **i32)
    pair_out = torch.empty(kvol * n, **i32)
    off_start = torch.empty(kvol + 1, **i32)
    tile_start = torch.empty(kvol + 1, **i32)
    nbytes = lib.ptv3_conv_pairs_workspace_bytes(n, kvol)
    ws = _lib.workspace(nbytes, dev)
    _lib.check(lib.ptv3_conv_pairs_build(_lib.ptr(nbr), _lib.ptr(row_order), n, kvol, _lib.ptr(pair_in),
                                         _lib.ptr(pair_out), _lib.ptr(off_start), _lib.ptr(tile_start),
                                         _lib.ptr(ws), nbytes, _lib.stream()), "ptv3_conv_pairs_build")
    return dict(pair_in=pair_in, pair_out=pair_out, off_start=off_start, tile_start=tile_start, n=n, kvol=kvol)


def subm_conv_pairs(feat, pairs, weight, bias=None):
    """Submanifold convolution over a pair list (bf16, coarse levels)."""
    _lib.require_cuda(feat, weight, bias)
    lib = _lib.load()
    feat = feat.contiguous()
    n, cin = feat.shape
    cout = weight.shape[0]
    out = torch.empty((n, cout), dtype=feat.dtype, device=feat.device)
    nbytes = n * cout * 8
    ws = _lib.workspace(nbytes, feat.device)
    with timed("subm_conv_pairs", 2.0 * n * pairs["kvol"] * cin * cout):
        _lib.check(lib.ptv3_subm_conv_pairs_fwd(
            _lib.ptr(feat), _lib.ptr(pairs["pair_in"]), _lib.ptr(pairs["pair_out"]), _lib.ptr(pairs["off_start"]),
            _lib.ptr(pairs["tile_start"]), _lib.ptr(weight.contiguous()), _lib.ptr(bias), _lib.ptr(out),
            _lib.ptr(ws), nbytes, n, cin, cout, pairs["kvol"], _lib.dtype_id(feat), _lib.stream()),
            "ptv3_subm_conv_pairs_fwd")
    return out


def linear_supported(k, n_out, residual_mode, dtype):
    return dtype in _lib.DTYPE_IDS and bool(
        _lib.load().ptv3_linear_supported(int(k), int(n_out), int(bool(residual_mode)), _lib.DTYPE_IDS[dtype]))


def linear(x, weight, bias, status=None):
    """out = x W^T + b on the tcgen05 path (see ptv3_linear_fwd)."""
    _lib.require_cuda(x, weight, bias)
    lib = _lib.load()
    x = x.contiguous()
    n, k = x.shape
    n_out = weight.shape[0]
    out = torch.empty((n, n_out), dtype=x.dtype, device=x.device)
    own = status is None
    if own:
        status = new_status(x.device)
    with timed("linear", 2.0 * n * k * n_out):
        _lib.check(lib.ptv3_linear_fwd(_lib.ptr(x), _lib.ptr(weight.contiguous()), _lib.ptr(bias), _lib.ptr(out), n, k,
                                       n_out, _lib.dtype_id(x), _lib.ptr(status), _lib.stream()), "ptv3_linear_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_linear_fwd")
    return out


def gemm_supported(k, n_out, dtype):
    return dtype in _lib.DTYPE_IDS and bool(_lib.load().ptv3_gemm_supported(int(k), int(n_out), _lib.DTYPE_IDS[dtype]))


def gemm(x, weight, bias=None, residual=None, gelu=False, status=None):
    """out = [residual +] act(x W^T + b) with streamed weights (see ptv3_gemm_fwd)."""
    _lib.require_cuda(x, weight, bias, residual)
    lib = _lib.load()
    x = x.contiguous()
    n, k = x.shape
    n_out = weight.shape[0]
    out = torch.empty((n, n_out), dtype=x.dtype, device=x.device)
    if residual is not None:
        residual = residual.contiguous()
        if residual.shape != out.shape or residual.dtype != x.dtype:
            raise ValueError("residual must be (n, n_out) in the feature dtype")
    own = status is None
    if own:
        status = new_status(x.device)
    with timed("gemm", 2.0 * n * k * n_out):
        _lib.check(lib.ptv3_gemm_fwd(_lib.ptr(x), _lib.ptr(weight.contiguous()), _lib.ptr(bias), _lib.ptr(residual),
                                     _lib.ptr(out), n, k, n_out, int(bool(gelu)), _lib.dtype_id(x), _lib.ptr(status),
                                     _lib.stream()), "ptv3_gemm_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_gemm_fwd")
    return out


def linear_ln(x, weight, bias, residual, ln1, ln2, status=None, want_sum=True):
    """(sum, normed) with y = x W^T + b, sum = residual + LN1(y) (or + y), normed = LN2(sum)."""
    _lib.require_cuda(x, weight, bias, residual)
    lib = _lib.load()
    x, residual = x.contiguous(), residual.contiguous()
    n, c = x.shape
    s = torch.empty_like(x) if want_sum else None
    y = torch.empty_like(x)
    own = status is None
    if own:
        status = new_status(x.device)
    w1, b1, e1 = (ln1.weight, ln1.bias, float(ln1.eps)) if ln1 is not None else (None, None, 0.0)
    with timed("linear_ln", 2.0 * n * c * c):
        _lib.check(lib.ptv3_linear_ln_fwd(_lib.ptr(x), _lib.ptr(weight.contiguous()), _lib.ptr(bias),
                                          _lib.ptr(residual), _lib.ptr(w1), _lib.ptr(b1), e1, _lib.ptr(s),
                                          _lib.ptr(ln2.weight), _lib.ptr(ln2.bias), float(ln2.eps), _lib.ptr(y), n, c,
                                          _lib.dtype_id(x), _lib.ptr(status), _lib.stream()), "ptv3_linear_ln_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_linear_ln_fwd")
    return s, y


def block_supported(channels, heads, hidden, dtype):
    return dtype in _lib.DTYPE_IDS and bool(
        _lib.load().ptv3_block_supported(int(channels), int(heads), int(hidden), _lib.DTYPE_IDS[dtype]))


def block(args, conv_in, feat, geometry, attention, status):
    """One transformer block through ptv3_block_fwd.

    args: a _lib.BlockArgs whose parameter pointers and static sizes the caller
    has filled in (and keeps alive); conv_in, feat: (N, C) bf16; geometry:
    dict(nbr, row_order) or a pair list of conv_pairs_build; attention:
    dict(order, pad, unpad, cu_seqlens, max_seqlen).  Returns the (N, C) output."""
    _lib.require_cuda(conv_in, feat, status)
    lib = _lib.load()
    conv_in, feat = conv_in.contiguous(), feat.contiguous()
    n = feat.shape[0]
    out = torch.empty_like(feat)
    args.n = n
    args.conv_in, args.feat, args.out = conv_in.data_ptr(), feat.data_ptr(), out.data_ptr()
    if "pair_in" in geometry:
        args.nbr = args.row_order = None
        args.pair_in, args.pair_out = geometry["pair_in"].data_ptr(), geometry["pair_out"].data_ptr()
        args.off_start, args.tile_start = geometry["off_start"].data_ptr(), geometry["tile_start"].data_ptr()
    else:
        args.pair_in = args.pair_out = args.off_start = args.tile_start = None
        args.nbr = geometry["nbr"].data_ptr()
        args.row_order = _lib.ptr(geometry["row_order"])
    args.order, args.pad, args.unpad = (attention["order"].data_ptr(), attention["pad"].data_ptr(),
                                        attention["unpad"].data_ptr())
    args.cu_seqlens = attention["cu_seqlens"].data_ptr()
    args.n_seq = attention["cu_seqlens"].numel() - 1
    args.max_seqlen = int(attention["max_seqlen"])
    args.status = status.data_ptr()
    nbytes = lib.ptv3_block_workspace_bytes(ctypes.byref(args))
    ws = _lib.workspace(nbytes, feat.device)
    args.workspace, args.workspace_bytes = ws.data_ptr(), nbytes
    C, H = args.channels, args.hidden
    with timed("block", 2.0 * n * (27 * C * C + 4 * C * C + 2 * C * H)):
        _lib.check(lib.ptv3_block_fwd(ctypes.byref(args), _lib.stream()), "ptv3_block_fwd")
    return out


def grid_coord(coord, grid_size):
    """coord (N, 3) float32 -> (grid_coord (N, 3) int32, origin (3,) float32):
    trunc((coord - coord.min(0)) / grid_size), model.py:94-96."""
    _lib.require_cuda(coord)
    lib = _lib.load()
    coord = coord.to(torch.float32).contiguous()
    n = coord.shape[0]
    grid = torch.empty((n, 3), dtype=torch.int32, device=coord.device)
    origin = torch.empty(3, dtype=torch.float32, device=coord.device)
    with timed("grid_coord", 36.0 * n):
        _lib.check(lib.ptv3_grid_coord(_lib.ptr(coord), n, float(grid_size), _lib.ptr(origin), _lib.ptr(grid),
                                       _lib.stream()), "ptv3_grid_coord")
    return grid, origin


def voxel_dedup(indices, offset=None, status=None):
    """indices (N, 4) int32 rows (scene, x, y, z) -> dict(keep (M,), point2voxel (N,),
    offset (scenes,) or None, m): the first point of every occupied voxel.  One host
    read (the number of voxels)."""
    _lib.require_cuda(indices, offset)
    lib = _lib.load()
    indices = indices.to(torch.int32).contiguous()
    n = indices.shape[0]
    dev = indices.device
    keep = torch.empty(n, dtype=torch.int64, device=dev)
    p2v = torch.empty(n, dtype=torch.int64, device=dev)
    n_scenes = 0 if offset is None else offset.numel()
    off_in = None if offset is None else offset.to(torch.int64).contiguous()
    new_offset = None if offset is None else torch.empty(n_scenes, dtype=torch.int64, device=dev)
    count = torch.zeros(1, dtype=torch.int64, device=dev)
    own = status is None
    if own:
        status = new_status(dev)
    nbytes = lib.ptv3_voxel_dedup_workspace_bytes(n)
    ws = _lib.workspace(nbytes, dev)
    with timed("voxel_dedup", 48.0 * n):
        _lib.check(lib.ptv3_voxel_dedup(_lib.ptr(indices), n, _lib.ptr(off_in), n_scenes, _lib.ptr(keep),
                                        _lib.ptr(p2v), _lib.ptr(new_offset), _lib.ptr(count), _lib.ptr(status),
                                        _lib.ptr(ws), nbytes, _lib.stream()), "ptv3_voxel_dedup")
    host = torch.cat([count, status.to(torch.int64)]).tolist()      # the one sync
    if own and host[1]:
        raise _lib.Ptv3Error("ptv3_voxel_dedup: device status 0x%x" % host[1])
    m = host[0]
    return dict(keep=keep[:m], point2voxel=p2v, offset=new_offset, m=m)


def seg_head(feat, weight, bias=None, want_logits=True, want_labels=True):
    """feat (N, C), weight (K, C) -> (logits (N, K) or None, labels (N,) int64 or None)."""
    _lib.require_cuda(feat, weight, bias)
    lib = _lib.load()
    feat = feat.contiguous()
    n, C = feat.shape
    K = weight.shape[0]
    logits = torch.empty((n, K), dtype=feat.dtype, device=feat.device) if want_logits else None
    labels = torch.empty(n, dtype=torch.int64, device=feat.device) if want_labels else None
    with timed("seg_head", 2.0 * n * C * K):
        _lib.check(lib.ptv3_seg_head_fwd(_lib.ptr(feat), _lib.ptr(weight.to(feat.dtype).contiguous()),
                                         _lib.ptr(None if bias is None else bias.to(feat.dtype).contiguous()),
                                         _lib.ptr(logits), _lib.ptr(labels), n, C, K, _lib.dtype_id(feat),
                                         _lib.stream()), "ptv3_seg_head_fwd")
    return logits, labels


def pool_stage_supported(c_in, c_out, dtype):
    """Whether a projection c_in -> c_out can go through the one-call stage transitions."""
    return dtype in _lib.DTYPE_IDS and bool(
        _lib.load().ptv3_pool_stage_supported(int(c_in), int(c_out), _lib.DTYPE_IDS[dtype]))


def pool_stage(x, weight, bias, coord, indices, idx_ptr, bn_scale=None, bn_shift=None, reduce="max", status=None):
    """SerializedPooling's feature side in one call (bf16): proj(x), segment reduction,
    BN + GELU, mean coordinate.  Returns (pooled feat (M, C_out), pooled coord or None)."""
    _lib.require_cuda(x, weight, bias, indices, idx_ptr)
    lib = _lib.load()
    x = x.contiguous()
    n, cin = x.shape
    cout = weight.shape[0]
    m = idx_ptr.numel() - 1
    out = torch.empty((m, cout), dtype=x.dtype, device=x.device)
    cout_coord = None
    if coord is not None:
        coord = coord.to(torch.float32).contiguous()
        cout_coord = torch.empty((m, 3), dtype=torch.float32, device=x.device)
    nbytes = lib.ptv3_pool_stage_workspace_bytes(n, cout)
    ws = _lib.workspace(nbytes, x.device)
    own = status is None
    if own:
        status = new_status(x.device)
    with timed("pool_stage", 2.0 * n * cin * cout):
        _lib.check(lib.ptv3_pool_stage_fwd(_lib.ptr(x), _lib.ptr(weight), _lib.ptr(bias), _lib.ptr(coord),
                                           _lib.ptr(indices), _lib.ptr(idx_ptr), n, m, cin, cout,
                                           _lib.ptr(bn_scale), _lib.ptr(bn_shift), _lib.ptr(out),
                                           _lib.ptr(cout_coord), REDUCE_IDS[reduce], _lib.dtype_id(x),
                                           _lib.ptr(status), _lib.ptr(ws), nbytes, _lib.stream()),
                   "ptv3_pool_stage_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_pool_stage_fwd")
    return out, cout_coord


def unpool_stage(skip_feat, child_feat, w_skip, b_skip, w_child, b_child, cluster, skip_scale, skip_shift,
                 child_scale, child_shift, status=None):
    """SerializedUnpooling in one call (bf16); returns (out, skip_act) as ops.unpool does."""
    _lib.require_cuda(skip_feat, child_feat, cluster)
    lib = _lib.load()
    skip_feat, child_feat = skip_feat.contiguous(), child_feat.contiguous()
    n, cs = skip_feat.shape
    m, cc = child_feat.shape
    cout = w_skip.shape[0]
    out = torch.empty((n, cout), dtype=skip_feat.dtype, device=skip_feat.device)
    act = torch.empty_like(out)
    nbytes = lib.ptv3_unpool_stage_workspace_bytes(n, m, cout)
    ws = _lib.workspace(nbytes, skip_feat.device)
    own = status is None
    if own:
        status = new_status(skip_feat.device)
    with timed("unpool_stage", 2.0 * cout * (n * cs + m * cc)):
        _lib.check(lib.ptv3_unpool_stage_fwd(_lib.ptr(skip_feat), _lib.ptr(child_feat), _lib.ptr(w_skip),
                                             _lib.ptr(b_skip), _lib.ptr(w_child), _lib.ptr(b_child),
                                             _lib.ptr(cluster), n, m, cs, cc, cout, _lib.ptr(skip_scale),
                                             _lib.ptr(skip_shift), _lib.ptr(child_scale), _lib.ptr(child_shift),
                                             _lib.ptr(out), _lib.ptr(act), _lib.dtype_id(skip_feat),
                                             _lib.ptr(status), _lib.ptr(ws), nbytes, _lib.stream()),
                   "ptv3_unpool_stage_fwd")
    if own:
        _lib.raise_on_status(status, "ptv3_unpool_stage_fwd")
    return out, act
