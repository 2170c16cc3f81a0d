"""ctypes bindings of the C ABI in include/scn_b200.h, taking torch CUDA tensors.

torch is used only for device memory and streams: every function passes raw device pointers
and torch's current stream to libscn_b200.so.
"""
import ctypes

import torch

from . import KERNEL_LIB

c_int, c_ll, c_f, c_p, c_sz = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t

SCN_OK = 0
LATTICE_SQUARE, LATTICE_TRIANGULAR = 0, 1
NOSIGMOID, RELU, VLEAKYRELU, LEAKYRELU, TANH, SOFTMAX, PRELU, SIGMOID = range(8)
PREC_AUTO, PREC_FP32, PREC_3XTF32, PREC_BF16, PREC_3XBF16, PREC_SPLIT = -1, 0, 1, 2, 3, 4
DEV_ERR_CAPACITY, DEV_ERR_KEY, DEV_ERR_DUPLICATE = 1, 2, 4

EXPORTS = [
    "scn_status_string", "scn_last_error", "scn_kernel_launch_count", "scn_device_supported", "scn_regions_cells",
    "scn_rules_workspace_bytes", "scn_rules_build", "scn_fmp_rules_workspace_bytes", "scn_fmp_rules_build", "scn_rules_static_scratch_bytes", "scn_rules_build_static", "scn_rules_chain_workspace_bytes", "scn_rules_chain_supported", "scn_rules_chain_build", "scn_rules_chain_resident_create", "scn_rules_chain_resident_destroy", "scn_rules_chain_resident_invalidate", "scn_rules_chain_resident_workspace_bytes", "scn_rules_chain_build_resident", "scn_terminal_rules_workspace_bytes",
    "scn_terminal_rules_build", "scn_conv_auto_precision", "scn_conv_nin_forward", "scn_conv_nin_forward_ws", "scn_conv_nin_forward_dyn", "scn_conv_nin_maxpool_forward", "scn_conv_nin_nin_forward", "scn_conv_nin_workspace_bytes", "scn_conv_packed_weight_bytes",
    "scn_conv_pack_weights", "scn_conv_tc_take_error", "scn_conv_tc_error_word", "scn_classifier_result_bytes", "scn_classifier_result", "scn_gather_forward", "scn_maxpool_forward",
    "scn_terminal_pool_forward", "scn_top_indices", "scn_activation_forward", "scn_background_rows",
    "scn_exchange_buffer_bytes", "scn_exchange_set_timeout_ms", "scn_exchange_alloc", "scn_exchange_free", "scn_exchange_open", "scn_exchange_close", "scn_exchange_publish", "scn_exchange_collect", "scn_exchange_step",
    "scn_mask_columns", "scn_sgd_update_masked", "scn_gather_columns", "scn_scatter_columns_axpy", "scn_sgemm_rowmajor", "scn_softmax_nll_backward", "scn_activation_backward", "scn_conv_nin_backward_weights", "scn_conv_nin_backward_weights_tc_bytes", "scn_conv_nin_backward_weights_tc", "scn_transpose_weights", "scn_gather_backward",
    "scn_maxpool_backward", "scn_terminal_pool_backward", "scn_sgd_update",
]


class Regions(ctypes.Structure):
    _fields_ = [(n, c_int) for n in ("lattice", "dim", "nIn", "nOut", "size", "stride", "minActive")]


class ChainLayer(ctypes.Structure):
    _fields_ = [("regions", Regions), ("d_out_keys", c_p), ("d_out_off", c_p), ("d_out_bg", c_p), ("d_rules", c_p),
                ("rows_out_capacity", c_int), ("d_result", c_p)]


class ScnError(RuntimeError):
    pass


_lib = None


def lib():
    """The kernel library; raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        try:
            L = ctypes.CDLL(KERNEL_LIB)
        except OSError as e:
            raise ScnError("libscn_b200.so is missing or unloadable (%s): run __graft_entry__.build()" % e)
        L.scn_status_string.restype = ctypes.c_char_p
        L.scn_status_string.argtypes = [c_int]
        L.scn_last_error.restype = ctypes.c_char_p
        L.scn_device_supported.restype = c_int
        L.scn_kernel_launch_count.restype = c_ll
        L.scn_conv_tc_error_word.restype = c_p
        L.scn_classifier_result_bytes.restype = c_sz
        L.scn_regions_cells.restype, L.scn_regions_cells.argtypes = c_int, [c_p]
        L.scn_exchange_buffer_bytes.restype, L.scn_exchange_buffer_bytes.argtypes = c_sz, [c_int, c_int]
        L.scn_exchange_set_timeout_ms.restype, L.scn_exchange_set_timeout_ms.argtypes = None, [c_int]
        L.scn_exchange_alloc.argtypes = [c_sz, c_p, c_p]
        L.scn_exchange_free.argtypes = [c_p]
        L.scn_exchange_open.argtypes = [c_p, c_p]
        L.scn_exchange_close.argtypes = [c_p]
        L.scn_exchange_publish.argtypes = [c_p, c_int, c_int, c_p, c_int, c_int, c_int, ctypes.c_uint, c_p]
        L.scn_exchange_collect.argtypes = [c_p, c_int, c_int, ctypes.c_uint, c_p, c_p, c_p, c_p]
        L.scn_exchange_step.argtypes = [c_p, ctypes.c_uint, c_p, c_p, c_p, c_p, c_int, c_int, c_p, c_int, c_int, c_int, ctypes.c_uint, c_p]
        L.scn_rules_workspace_bytes.restype = c_sz
        L.scn_rules_workspace_bytes.argtypes = [c_p, c_int, c_int]
        L.scn_rules_build.argtypes = [c_p, c_int, c_p, c_p, c_p, c_int, c_p, c_p, c_p, c_p, c_int, c_p, c_p, c_sz, c_p]
        L.scn_fmp_rules_workspace_bytes.restype = c_sz
        L.scn_fmp_rules_workspace_bytes.argtypes = [c_int] * 6
        L.scn_fmp_rules_build.argtypes = [c_int] * 6 + [c_p, c_p, c_p, c_p, c_int, c_p, c_p, c_p, c_p, c_int, c_p, c_p, c_sz, c_p]
        L.scn_rules_static_scratch_bytes.restype = c_sz
        L.scn_rules_build_static.argtypes = [c_p, c_int, c_p, c_p, c_p, c_int, c_p, c_p, c_p, c_p, c_int, c_p, c_p]
        L.scn_rules_chain_workspace_bytes.restype = c_sz
        L.scn_rules_chain_workspace_bytes.argtypes = [c_int, c_int]
        L.scn_rules_chain_supported.argtypes = [c_p, c_int, c_int, c_int, c_int]
        L.scn_rules_chain_build.argtypes = [c_p, c_int, c_int, c_p, c_p, c_p, c_int, c_int, c_p, c_sz, c_p]
        L.scn_terminal_rules_workspace_bytes.restype = c_sz
        L.scn_terminal_rules_workspace_bytes.argtypes = [c_int] * 4
        L.scn_terminal_rules_build.argtypes = [c_int, c_int, c_int, c_p, c_p, c_p, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p, c_sz, c_p]
        L.scn_conv_nin_forward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p, c_p, c_p, c_int, c_f, c_int, c_int, c_p, c_p]
        L.scn_conv_nin_forward_dyn.argtypes = [c_p, c_p, c_int, c_p, c_int, c_int, c_p, c_p, c_p, c_int, c_f, c_int, c_p, c_p]
        L.scn_conv_nin_maxpool_forward.argtypes = [c_p, c_p, c_int, c_int, c_p, c_p, c_p, c_int, c_f, c_int, c_p, c_int, c_int, c_p, c_int, c_p, c_p, c_p, c_sz, c_p]
        L.scn_conv_nin_nin_forward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p, c_p, c_int, c_f, c_int, c_p, c_p, c_p, c_int, c_f, c_int, c_p, c_p, c_p, c_sz, c_p]
        L.scn_conv_nin_forward_ws.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p, c_p, c_p, c_int, c_f, c_int, c_int, c_p, c_p, c_sz, c_p]
        L.scn_conv_nin_workspace_bytes.restype = c_sz
        L.scn_conv_nin_workspace_bytes.argtypes = [c_int] * 5
        L.scn_conv_packed_weight_bytes.restype = c_sz
        L.scn_conv_packed_weight_bytes.argtypes = [c_int, c_int, c_int]
        L.scn_conv_pack_weights.argtypes = [c_p, c_int, c_int, c_int, c_p, c_p]
        L.scn_gather_forward.argtypes = [c_p, c_p, c_ll, c_int, c_p, c_p]
        L.scn_maxpool_forward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p, c_p]
        L.scn_terminal_pool_forward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p]
        L.scn_top_indices.argtypes = [c_p, c_int, c_int, c_int, c_p, c_p]
        L.scn_activation_forward.argtypes = [c_p, c_p, c_int, c_int, c_int, c_p, c_p]
        L.scn_background_rows.argtypes = [c_p, c_p, c_int, c_p, c_p]
        _lib = L
    return _lib


def check(status):
    if status != SCN_OK:
        L = lib()
        raise ScnError("%s: %s" % (L.scn_status_string(status).decode(), L.scn_last_error().decode()))


def _ptr(t):
    return None if t is None else c_p(t.data_ptr())


def _stream():
    return c_p(torch.cuda.current_stream().cuda_stream)


def _i32(t):
    assert t.is_cuda and t.dtype == torch.int32 and t.is_contiguous()
    return t


def _f32(t):
    assert t.is_cuda and t.dtype == torch.float32 and t.is_contiguous()
    return t


def regions(lattice, dim, nIn, nOut, size, stride, minActive=1):
    return Regions(lattice, dim, nIn, nOut, size, stride, minActive)


def rules_build(R, keys, off, bg, rows_out_capacity, rows_in_bound=None):
    """scn_rules_build over torch int32 CUDA tensors.  Returns the raw outputs at capacity
    size plus d_result; nothing is synchronised."""
    L = lib()
    batch = bg.numel()
    rows_in_bound = keys.numel() if rows_in_bound is None else rows_in_bound
    sd = L.scn_regions_cells(ctypes.byref(R))
    if sd < 0:
        raise ScnError("invalid argument: %s" % L.scn_last_error().decode())
    dev = keys.device
    ws_bytes = L.scn_rules_workspace_bytes(ctypes.byref(R), batch, rows_in_bound)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    out_keys = torch.empty(max(rows_out_capacity, 1), dtype=torch.int32, device=dev)
    out_off = torch.empty(batch + 1, dtype=torch.int32, device=dev)
    out_bg = torch.empty(batch, dtype=torch.int32, device=dev)
    rules = torch.empty(max(rows_out_capacity, 1) * sd, dtype=torch.int32, device=dev)
    result = torch.empty(4, dtype=torch.int32, device=dev)
    check(L.scn_rules_build(ctypes.byref(R), batch, _ptr(_i32(keys)), _ptr(_i32(off)), _ptr(_i32(bg)), rows_in_bound,
                            _ptr(out_keys), _ptr(out_off), _ptr(out_bg), _ptr(rules), rows_out_capacity, _ptr(result),
                            _ptr(ws), ws_bytes, _stream()))
    return dict(out_keys=out_keys, out_off=out_off, out_bg=out_bg, rules=rules, result=result, sd=sd, workspace=ws)


def fmp_rules_build(dim, nIn, nOut, poolSize, overlapping, ticks, keys, off, bg, rows_out_capacity):
    """scn_fmp_rules_build: ticks is an int32 CUDA tensor [batch, dim, 2*nOut + 2*nIn]."""
    L = lib()
    batch = bg.numel()
    dev = keys.device
    sd = poolSize ** dim
    ws_bytes = L.scn_fmp_rules_workspace_bytes(dim, nIn, nOut, poolSize, batch, keys.numel())
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    out_keys = torch.empty(max(rows_out_capacity, 1), dtype=torch.int32, device=dev)
    out_off = torch.empty(batch + 1, dtype=torch.int32, device=dev)
    out_bg = torch.empty(batch, dtype=torch.int32, device=dev)
    rules = torch.empty(max(rows_out_capacity, 1) * sd, dtype=torch.int32, device=dev)
    result = torch.empty(4, dtype=torch.int32, device=dev)
    check(L.scn_fmp_rules_build(dim, nIn, nOut, poolSize, int(overlapping), batch, _ptr(_i32(ticks)), _ptr(_i32(keys)), _ptr(_i32(off)),
                                _ptr(_i32(bg)), keys.numel(), _ptr(out_keys), _ptr(out_off), _ptr(out_bg), _ptr(rules),
                                rows_out_capacity, _ptr(result), _ptr(ws), ws_bytes, _stream()))
    return dict(out_keys=out_keys, out_off=out_off, out_bg=out_bg, rules=rules, result=result, sd=sd, workspace=ws)


def terminal_rules_build(dim, spatial_size, keys, off, bg, S):
    L = lib()
    batch = bg.numel()
    dev = keys.device
    ws_bytes = L.scn_terminal_rules_workspace_bytes(dim, spatial_size, batch, keys.numel())
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
    out_keys = torch.empty(batch, dtype=torch.int32, device=dev)
    out_off = torch.empty(batch + 1, dtype=torch.int32, device=dev)
    out_bg = torch.empty(batch, dtype=torch.int32, device=dev)
    rules = torch.empty(batch * S, dtype=torch.int32, device=dev)
    result = torch.empty(4, dtype=torch.int32, device=dev)
    check(L.scn_terminal_rules_build(dim, spatial_size, batch, _ptr(_i32(keys)), _ptr(_i32(off)), _ptr(_i32(bg)),
                                     keys.numel(), S, _ptr(out_keys), _ptr(out_off), _ptr(out_bg), _ptr(rules),
                                     _ptr(result), _ptr(ws), ws_bytes, _stream()))
    return dict(out_keys=out_keys, out_off=out_off, out_bg=out_bg, rules=rules, result=result, workspace=ws)


def pack_weights(W, precision):
    L = lib()
    K, N = W.shape
    nbytes = L.scn_conv_packed_weight_bytes(K, N, precision)
    if nbytes == 0:
        raise ScnError("unsupported configuration: no packed layout for K=%d N=%d precision=%d" % (K, N, precision))
    packed = torch.empty(nbytes, dtype=torch.uint8, device=W.device)
    check(L.scn_conv_pack_weights(_ptr(_f32(W)), K, N, precision, _ptr(packed), _stream()))
    return packed


def conv_nin_forward(feat, rules, fs, W, B, prelu=None, p=1.0, act=NOSIGMOID, precision=PREC_FP32, packed=None,
                     rows_out=None, split_k=True):
    """rules: int32 [rows_out*fs] or None (plain NiN, fs == 1)."""
    L = lib()
    nIn = feat.shape[1]
    K, N = W.shape
    assert K == fs * nIn
    if rows_out is None:
        rows_out = feat.shape[0] if rules is None else rules.numel() // fs
    out = torch.empty((rows_out, N), dtype=torch.float32, device=feat.device)
    ws_bytes = L.scn_conv_nin_workspace_bytes(rows_out, fs, nIn, N, precision) if (split_k and packed is not None) else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=feat.device) if ws_bytes else None
    check(L.scn_conv_nin_forward_ws(_ptr(_f32(feat)), _ptr(rules), rows_out, fs, nIn, _ptr(_f32(W)), _ptr(packed),
                                    _ptr(_f32(B)), _ptr(prelu), N, p, act, precision, _ptr(out), _ptr(ws), ws_bytes, _stream()))
    return out


def gather_forward(feat, rules):
    nIn = feat.shape[1]
    out = torch.empty((rules.numel(), nIn), dtype=torch.float32, device=feat.device)
    check(lib().scn_gather_forward(_ptr(_f32(feat)), _ptr(_i32(rules)), rules.numel(), nIn, _ptr(out), _stream()))
    return out


def maxpool_forward(feat, rules, sd):
    C = feat.shape[1]
    rows_out = rules.numel() // sd
    out = torch.empty((rows_out, C), dtype=torch.float32, device=feat.device)
    ch = torch.empty((rows_out, C), dtype=torch.int32, device=feat.device)
    check(lib().scn_maxpool_forward(_ptr(_f32(feat)), _ptr(_i32(rules)), rows_out, sd, C, _ptr(out), _ptr(ch), _stream()))
    return out, ch


def terminal_pool_forward(feat, rules, S):
    C = feat.shape[1]
    batch = rules.numel() // S
    out = torch.empty((batch, C), dtype=torch.float32, device=feat.device)
    check(lib().scn_terminal_pool_forward(_ptr(_f32(feat)), _ptr(_i32(rules)), batch, S, C, _ptr(out), _stream()))
    return out


def top_indices(probs, nTop):
    rows, nClasses = probs.shape
    top = torch.empty((rows, nTop), dtype=torch.int32, device=probs.device)
    check(lib().scn_top_indices(_ptr(_f32(probs)), rows, nClasses, nTop, _ptr(top), _stream()))
    return top


def activation_forward(x, act, prelu=None):
    rows, N = x.shape
    out = torch.empty_like(x)
    check(lib().scn_activation_forward(_ptr(_f32(x)), _ptr(out), rows, N, act, _ptr(prelu), _stream()))
    return out


def classifier_result(probs, nTop):
    """scn_classifier_result -> (probabilities, top, tc_error) unpacked from the one block the kernel writes."""
    L = lib()
    rows, nClasses = probs.shape
    L.scn_classifier_result_bytes.restype = c_sz
    nbytes = L.scn_classifier_result_bytes(rows, nClasses, nTop)
    block = torch.empty(nbytes // 4, dtype=torch.int32, device=probs.device)
    check(L.scn_classifier_result(_ptr(_f32(probs)), rows, nClasses, nTop, _ptr(block), _stream()))
    host = block.cpu()
    p = host[: rows * nClasses].view(torch.float32).reshape(rows, nClasses)
    t = host[rows * nClasses: rows * nClasses + rows * nTop].reshape(rows, nTop)
    return p, t, int(host[-1])


def kernel_launch_count():
    return int(lib().scn_kernel_launch_count())


def conv_tc_take_error():
    return int(lib().scn_conv_tc_take_error())


def rules_build_static(R, keys, off, bg, rows_out_capacity, out=None):
    """scn_rules_build_static: the rule build whose scratch is the library's fixed device array,
    for callers that must not allocate.  Pass `out` (a dict from an earlier call) to reuse its
    output tensors, so that the call itself creates no tensor at all."""
    L = lib()
    batch = bg.numel()
    sd = L.scn_regions_cells(ctypes.byref(R))
    if sd < 0:
        raise ScnError("invalid argument: %s" % L.scn_last_error().decode())
    if out is None:
        dev = keys.device
        out = dict(out_keys=torch.empty(max(rows_out_capacity, 1), dtype=torch.int32, device=dev),
                   out_off=torch.empty(batch + 1, dtype=torch.int32, device=dev),
                   out_bg=torch.empty(batch, dtype=torch.int32, device=dev),
                   rules=torch.empty(max(rows_out_capacity, 1) * sd, dtype=torch.int32, device=dev),
                   result=torch.empty(4, dtype=torch.int32, device=dev), sd=sd)
    check(L.scn_rules_build_static(ctypes.byref(R), batch, _ptr(_i32(keys)), _ptr(_i32(off)), _ptr(_i32(bg)), keys.numel(),
                                   _ptr(out["out_keys"]), _ptr(out["out_off"]), _ptr(out["out_bg"]), _ptr(out["rules"]),
                                   rows_out_capacity, _ptr(out["result"]), _stream()))
    return out


def rules_chain_build(regions_list, keys, off, bg, max_rows_per_sample, capacities, rows_hint=0):
    """scn_rules_chain_build: all geometry layers of a network in one kernel.  Returns one
    output dict per layer (as rules_build), or None if the samples are too large for it."""
    L = lib()
    batch = bg.numel()
    dev = keys.device
    n = len(regions_list)
    arr = (ChainLayer * n)()
    outs = []
    for i, (R, cap) in enumerate(zip(regions_list, capacities)):
        sd = L.scn_regions_cells(ctypes.byref(R))
        if sd < 0:
            raise ScnError("invalid argument: %s" % L.scn_last_error().decode())
        o = dict(out_keys=torch.empty(max(cap, 1), dtype=torch.int32, device=dev),
                 out_off=torch.empty(batch + 1, dtype=torch.int32, device=dev),
                 out_bg=torch.empty(batch, dtype=torch.int32, device=dev),
                 rules=torch.empty(max(cap, 1) * sd, dtype=torch.int32, device=dev),
                 result=torch.empty(4, dtype=torch.int32, device=dev), sd=sd)
        outs.append(o)
        arr[i].regions = R
        arr[i].d_out_keys, arr[i].d_out_off, arr[i].d_out_bg = o["out_keys"].data_ptr(), o["out_off"].data_ptr(), o["out_bg"].data_ptr()
        arr[i].d_rules, arr[i].rows_out_capacity, arr[i].d_result = o["rules"].data_ptr(), cap, o["result"].data_ptr()
    if not L.scn_rules_chain_supported(arr, n, batch, max_rows_per_sample, rows_hint):
        return None
    nbytes = L.scn_rules_chain_workspace_bytes(n, batch)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    check(L.scn_rules_chain_build(arr, n, batch, _ptr(_i32(keys)), _ptr(_i32(off)), _ptr(_i32(bg)), max_rows_per_sample,
                                  rows_hint, _ptr(ws), nbytes, _stream()))
    for o in outs:
        o["workspace"] = ws
    return outs


class ResidentChain:
    """scn_rules_chain_build_resident: a chain of geometry layers whose device state stays with this object from call to
    call, so that in steady state the kernel is the only stream operation.  Two sets of result records alternate; each
    build() returns the per-layer output dicts of the set it used (valid until the call after next)."""

    def __init__(self, regions_list, batch, capacities, device):
        L = lib()
        L.scn_rules_chain_resident_create.restype = c_p
        L.scn_rules_chain_resident_workspace_bytes.restype = c_sz
        self.L, self.n, self.batch = L, len(regions_list), batch
        self.state = c_p(L.scn_rules_chain_resident_create())
        self.results = torch.zeros((2, 4 * self.n), dtype=torch.int32, device=device)
        self.arr, self.outs = [], []
        for phase in range(2):
            arr = (ChainLayer * self.n)()
            outs = []
            for i, (R, cap) in enumerate(zip(regions_list, capacities)):
                sd = L.scn_regions_cells(ctypes.byref(R))
                o = dict(out_keys=torch.empty(max(cap, 1), dtype=torch.int32, device=device),
                         out_off=torch.empty(batch + 1, dtype=torch.int32, device=device),
                         out_bg=torch.empty(batch, dtype=torch.int32, device=device),
                         rules=torch.empty(max(cap, 1) * sd, dtype=torch.int32, device=device),
                         result=self.results[phase, 4 * i: 4 * i + 4], sd=sd)
                outs.append(o)
                arr[i].regions = R
                arr[i].d_out_keys, arr[i].d_out_off, arr[i].d_out_bg = o["out_keys"].data_ptr(), o["out_off"].data_ptr(), o["out_bg"].data_ptr()
                arr[i].d_rules, arr[i].rows_out_capacity, arr[i].d_result = o["rules"].data_ptr(), cap, o["result"].data_ptr()
            self.arr.append(arr)
            self.outs.append(outs)
        self.nbytes = L.scn_rules_chain_resident_workspace_bytes(self.n, batch)
        self.ws = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.phase = 0
        self.bg = torch.empty(batch, dtype=torch.int32, device=device)

    def __del__(self):
        try:
            self.L.scn_rules_chain_resident_destroy(self.state)
        except Exception:
            pass

    def build(self, keys, off, bg, max_rows_per_sample, rows_hint=0):
        """bg None: the kernel finds the background rows (returned as self.bg)."""
        p = self.phase
        self.phase ^= 1
        check(self.L.scn_rules_chain_build_resident(self.state, self.arr[p], self.n, self.batch, _ptr(_i32(keys)), _ptr(_i32(off)),
                                                    None if bg is None else _ptr(_i32(bg)), _ptr(self.bg), max_rows_per_sample, rows_hint,
                                                    _ptr(self.ws), self.nbytes, p, _ptr(self.results[1 - p]), 4 * self.n, _stream()))
        return self.outs[p]


def conv_nin_forward_dyn(feat, rules, fs, W, B, d_rows, rows_bound, prelu=None, p=1.0, act=NOSIGMOID, packed=None, precision=PREC_3XTF32):
    """scn_conv_nin_forward_dyn: the split tensor-core kernel (weights packed for `precision`: PREC_3XTF32 or PREC_SPLIT) with
    its row count read from the int32 CUDA tensor d_rows (clamped to rows_bound).  Returns [rows_bound x N]; rows past the
    count are left untouched."""
    L = lib()
    K, N = W.shape
    nIn = K // fs
    out = torch.zeros((rows_bound, N), dtype=torch.float32, device=feat.device)
    check(L.scn_conv_nin_forward_dyn(_ptr(_f32(feat)), None if rules is None else _ptr(_i32(rules)), rows_bound, _ptr(_i32(d_rows)), fs, nIn,
                                     _ptr(packed), _ptr(_f32(B)), None if prelu is None else _ptr(_f32(prelu)), N, p, act, _ptr(out), precision, _stream()))
    return out


def conv_nin_maxpool_forward(feat, rules, fs, W, B, pool_rules, cells, prelu=None, p=1.0, act=NOSIGMOID, packed=None, d_rows=None,
                             rows_unpooled=0, split_k=False, precision=PREC_3XTF32):
    """scn_conv_nin_maxpool_forward -> (pooled [rows_pool x N], choices).  split_k: hand over the workspace with which a
    layer of few tiles splits K (the pooling then happens where the partial sums are added); needs rows_unpooled."""
    L = lib()
    K, N = W.shape
    rows_pool = pool_rules.numel() // cells
    ws_bytes = L.scn_conv_nin_workspace_bytes(rows_unpooled, fs, K // fs, N, precision) if (split_k and rows_unpooled) else 0
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=feat.device) if ws_bytes else None
    out = torch.zeros((rows_pool, N), dtype=torch.float32, device=feat.device)
    choices = torch.full((rows_pool, N), -7, dtype=torch.int32, device=feat.device)
    check(L.scn_conv_nin_maxpool_forward(_ptr(_f32(feat)), _ptr(_i32(rules)), fs, K // fs, _ptr(packed), _ptr(_f32(B)),
                                         None if prelu is None else _ptr(_f32(prelu)), N, p, act, _ptr(_i32(pool_rules)), cells, rows_pool,
                                         None if d_rows is None else _ptr(_i32(d_rows)), rows_unpooled, _ptr(out), _ptr(choices),
                                         _ptr(ws), ws_bytes, precision, _stream()))
    return out, choices


def conv_nin_nin_forward(feat, rules, fs, W, B, W2, B2, prelu=None, p=1.0, act=NOSIGMOID, p2=1.0, act2=SOFTMAX, packed=None,
                         precision=PREC_3XTF32):
    """scn_conv_nin_nin_forward -> (first layer's output [rows x N], second's [rows x N2])."""
    L = lib()
    K, N = W.shape
    N2 = W2.shape[1]
    rows = feat.shape[0] if rules is None else rules.numel() // fs
    mid = torch.empty((rows, N), dtype=torch.float32, device=feat.device)
    out = torch.empty((rows, N2), dtype=torch.float32, device=feat.device)
    ws_bytes = L.scn_conv_nin_workspace_bytes(rows, fs, K // fs, N, precision)
    ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=feat.device)
    check(L.scn_conv_nin_nin_forward(_ptr(_f32(feat)), None if rules is None else _ptr(_i32(rules)), rows, fs, K // fs, _ptr(packed), _ptr(_f32(B)),
                                     None if prelu is None else _ptr(_f32(prelu)), N, p, act, _ptr(_f32(W2)), _ptr(_f32(B2)), None, N2, p2, act2,
                                     _ptr(mid), _ptr(out), _ptr(ws), ws_bytes, precision, _stream()))
    return mid, out


def background_rows(keys, off):
    batch = off.numel() - 1
    bg = torch.empty(batch, dtype=torch.int32, device=keys.device)
    check(lib().scn_background_rows(_ptr(_i32(keys)), _ptr(_i32(off)), batch, _ptr(bg), _stream()))
    return bg


# ---------------------------------------------------------------------------------------------- backward pass
def softmax_nll_backward(probs, labels):
    rows, C = probs.shape
    d = torch.empty_like(probs)
    check(lib().scn_softmax_nll_backward(_ptr(_f32(probs)), _ptr(_i32(labels)), rows, C, _ptr(d), _stream()))
    return d


def activation_backward(out_features, d, act, prelu=None):
    """-> (d * f'(.) as a new tensor, slope gradient or None)."""
    rows, N = out_features.shape
    d = d.clone()
    dpr = torch.zeros(N, dtype=torch.float32, device=d.device) if act == PRELU else None
    check(lib().scn_activation_backward(_ptr(_f32(out_features)), _ptr(d), rows, N, act, _ptr(prelu), _ptr(dpr), _stream()))
    return d, dpr


def conv_nin_backward_weights(feat, rules, fs, dout):
    """-> (dW [(fs*nIn) x N], dB [N])."""
    nIn = feat.shape[1]
    rows, N = dout.shape
    K = fs * nIn if rules is not None else nIn
    dW = torch.empty((K, N), dtype=torch.float32, device=dout.device)
    dB = torch.empty(N, dtype=torch.float32, device=dout.device)
    check(lib().scn_conv_nin_backward_weights(_ptr(_f32(feat)), None if rules is None else _ptr(_i32(rules)), rows, fs if rules is not None else 1,
                                              nIn, _ptr(_f32(dout)), N, _ptr(dW), _ptr(dB), _stream()))
    return dW, dB


def conv_nin_backward_weights_tc(feat, rules, fs, dout):
    """The same on the tensor cores -> (dW, dB); raises ScnError (unsupported configuration) for shapes it does not take."""
    nIn = feat.shape[1]
    rows, N = dout.shape
    f = fs if rules is not None else 1
    K = f * nIn
    L = lib()
    L.scn_conv_nin_backward_weights_tc_bytes.restype = c_sz
    nbytes = L.scn_conv_nin_backward_weights_tc_bytes(rows, f, nIn, N)
    if not nbytes:
        raise ScnError("unsupported configuration: the tensor-core weight gradient does not take rows=%d N=%d" % (rows, N))
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dout.device)
    dW = torch.empty((K, N), dtype=torch.float32, device=dout.device)
    dB = torch.empty(N, dtype=torch.float32, device=dout.device)
    check(L.scn_conv_nin_backward_weights_tc(_ptr(_f32(feat)), None if rules is None else _ptr(_i32(rules)), rows, f, nIn, _ptr(_f32(dout)), N,
                                             _ptr(dW), _ptr(dB), _ptr(ws), c_sz(nbytes), _stream()))
    return dW, dB


def transpose_weights(W):
    K, N = W.shape
    Wt = torch.empty((N, K), dtype=torch.float32, device=W.device)
    check(lib().scn_transpose_weights(_ptr(_f32(W)), K, N, _ptr(Wt), _stream()))
    return Wt


def gather_backward(dconv, rules, nIn, rows_in):
    din = torch.empty((rows_in, nIn), dtype=torch.float32, device=dconv.device)
    check(lib().scn_gather_backward(_ptr(_f32(dconv)), _ptr(_i32(rules)), c_ll(rules.numel()), nIn, _ptr(din), c_ll(rows_in), _stream()))
    return din


def maxpool_backward(dout, choices, n_in):
    din = torch.empty(n_in, dtype=torch.float32, device=dout.device)
    check(lib().scn_maxpool_backward(_ptr(_f32(dout)), _ptr(_i32(choices)), c_ll(dout.numel()), _ptr(din), c_ll(n_in), _stream()))
    return din


def terminal_pool_backward(dout, rules, S, rows_in):
    batch, C = dout.shape
    din = torch.empty((rows_in, C), dtype=torch.float32, device=dout.device)
    check(lib().scn_terminal_pool_backward(_ptr(_f32(dout)), _ptr(_i32(rules)), batch, S, C, _ptr(din), c_ll(rows_in), _stream()))
    return din


def sgd_update(w, m, d, lr, momentum, keep_positive=False):
    """In place on w and m."""
    check(lib().scn_sgd_update(_ptr(w), _ptr(m), _ptr(_f32(d)), c_ll(w.numel()), c_f(lr), c_f(momentum), int(keep_positive), _stream()))


def mask_columns(x, mask):
    """In place: x[r, n] = 0 where mask[n] == 0 (the features a training batch drops)."""
    rows, N = x.shape
    check(lib().scn_mask_columns(_ptr(x), c_ll(rows), N, _ptr(_f32(mask)), _stream()))


def sgd_update_masked(w, m, d, row_mask, row_period, col_mask, lr, momentum, keep_positive=False):
    """scn_sgd_update on the entries of w [rows x N] whose row mask (index row % row_period) and column mask are non-zero;
    either mask may be None.  In place on w and m."""
    rows, N = w.shape
    check(lib().scn_sgd_update_masked(_ptr(w), _ptr(m), _ptr(_f32(d)), c_ll(rows), N, _ptr(_f32(row_mask)) if row_mask is not None else None,
                                      int(row_period), _ptr(_f32(col_mask)) if col_mask is not None else None, c_f(lr), c_f(momentum),
                                      int(keep_positive), _stream()))


def sgemm_rowmajor(A, B, C, l, m, r, alpha=1.0, beta=0.0, trans_a=False, trans_b=False):
    """C[l x r] = alpha * op(A) op(B) + beta * C (in place on C)."""
    check(lib().scn_sgemm_rowmajor(int(trans_a), int(trans_b), _ptr(_f32(A)), _ptr(_f32(B)), _ptr(_f32(C)), l, m, r, c_f(alpha), c_f(beta), _stream()))


class ExchangeBuffer:
    """One rank's buffer of the result exchange (scn_exchange_alloc): blocks of at most cap_floats floats from each
    of `world` ranks.  `handle` is what another process of the node passes to ExchangeBuffer.open()."""

    def __init__(self, world, cap_floats):
        self.world, self.cap_floats = world, cap_floats
        nbytes = lib().scn_exchange_buffer_bytes(world, cap_floats)
        if not nbytes:
            raise ScnError("bad exchange sizes")
        p, h = c_p(), (ctypes.c_ubyte * 64)()
        check(lib().scn_exchange_alloc(c_sz(nbytes), ctypes.byref(p), h))
        self.ptr, self.handle = p.value, bytes(h)

    def free(self):
        if self.ptr:
            check(lib().scn_exchange_free(c_p(self.ptr)))
            self.ptr = None

    @staticmethod
    def open(handle):
        p = c_p()
        check(lib().scn_exchange_open((ctypes.c_ubyte * 64).from_buffer_copy(handle), ctypes.byref(p)))
        return p.value

    @staticmethod
    def close(ptr):
        check(lib().scn_exchange_close(c_p(ptr)))


def exchange_set_timeout_ms(ms):
    lib().scn_exchange_set_timeout_ms(int(ms))


def exchange_publish(block, rows, peers, rank, cap_floats, step):
    """block: float32 CUDA tensor (this rank's results of `step`); peers: every rank's buffer pointer."""
    arr = (c_p * len(peers))(*peers)
    check(lib().scn_exchange_publish(_ptr(_f32(block)), block.numel(), rows, arr, len(peers), rank, cap_floats, step, _stream()))


def exchange_collect(local_ptr, world, cap_floats, step, out=None, rows=None, status=None):
    """-> (out[world, cap_floats], rows[world], status[1]) once every rank's block of `step` has arrived or timed out."""
    dev = torch.device("cuda", torch.cuda.current_device())
    out = torch.zeros((world, cap_floats), dtype=torch.float32, device=dev) if out is None else out
    rows = torch.full((world,), -1, dtype=torch.int32, device=dev) if rows is None else rows
    status = torch.zeros(1, dtype=torch.int32, device=dev) if status is None else status
    check(lib().scn_exchange_collect(c_p(local_ptr), world, cap_floats, step, _ptr(out), _ptr(rows), _ptr(status), _stream()))
    return out, rows, status
