"""ctypes bindings of include/scn_b200_net.h: networks built from the C++ classes that keep
the reference's names (SparseConvNetCUDA and its layers), driven from Python.

torch supplies device buffers and the stream; all arithmetic runs in libscn_b200.so.
"""
import ctypes

import numpy as np
import torch

from . import HOST_LIB, abi

c_int, c_ll, c_f, c_p, c_d = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p, ctypes.c_double

EXPORTS = [
    "scn_net_last_error", "scn_net_create", "scn_net_destroy", "scn_net_addLeNetLayerMP", "scn_net_addLeNetLayerFMP", "scn_net_seed_fmp", "scn_net_set_pool_fusion",
    "scn_net_addTerminalPoolingLayer", "scn_net_addSoftmaxLayer", "scn_net_DeepCNet", "scn_net_named", "scn_net_n_layers",
    "scn_net_input_spatial_size", "scn_net_layer_info", "scn_net_set_weights", "scn_net_load_weights",
    "scn_net_save_weights", "scn_net_set_precision", "scn_net_forward_host", "scn_net_forward_device",
    "scn_net_copy_probs_device", "scn_net_train_batch", "scn_net_get_weights", "scn_net_iface_dfeatures", "scn_net_iface_sizes", "scn_net_iface_fetch", "scn_net_take_multiply_adds", "scn_net_enable_timing",
    "scn_net_layer_times", "scn_net_process_dataset", "scn_host_vectorTopIndices",
    "scn_net_exchange_create", "scn_net_exchange_buffer", "scn_net_exchange_connect", "scn_net_exchange_connect_local", "scn_net_exchange_destroy",
    "scn_net_forward_host_exchange", "scn_net_exchange_flush", "scn_net_exchange_step_device",
    "scn_net_forward_host_begin", "scn_net_forward_host_end", "scn_net_rescale_batch", "scn_net_addIndexLearnerLayer", "scn_net_index_learner_batch", "scn_net_set_dropout_features", "scn_net_iface_present",
]

LAYER_KEYS = ("type", "size", "stride", "minActive", "nIn", "nOut", "fs", "act", "inSpatial", "outSpatial")
L_CONV, L_CONV_TRI, L_NIN, L_MAXPOOL, L_MAXPOOL_TRI, L_TERMINAL = range(6)

_lib = None


def _current_stream():
    """torch's current stream as a cudaStream_t.  torch's default stream has handle 0, which
    the library would read as "create your own": name the legacy default stream explicitly."""
    h = torch.cuda.current_stream().cuda_stream
    return c_p(h if h else 1)  # 1 == cudaStreamLegacy


def lib():
    global _lib
    if _lib is None:
        abi.lib()  # the host library links against the kernel library
        try:
            L = ctypes.CDLL(HOST_LIB)
        except OSError as e:
            raise abi.ScnError("libscn_b200_host.so is missing or unloadable (%s): run __graft_entry__.build()" % e)
        L.scn_net_last_error.restype = ctypes.c_char_p
        L.scn_net_create.restype, L.scn_net_create.argtypes = c_p, [c_int] * 5 + [c_p]
        L.scn_net_destroy.argtypes = [c_p]
        L.scn_net_addLeNetLayerMP.argtypes = [c_p] + [c_int] * 6 + [c_f, c_int]
        L.scn_net_addLeNetLayerFMP.argtypes = [c_p] + [c_int] * 5 + [c_f, c_int, c_f, c_int]
        L.scn_net_seed_fmp.argtypes = [c_p, ctypes.c_uint]
        L.scn_net_set_pool_fusion.argtypes = [c_p, c_int]
        L.scn_net_addTerminalPoolingLayer.argtypes = [c_p, c_int]
        L.scn_net_addSoftmaxLayer.argtypes = [c_p]
        L.scn_net_DeepCNet.restype = c_p
        L.scn_net_DeepCNet.argtypes = [c_int] * 6 + [c_f, c_int, c_p]
        L.scn_net_named.restype = c_p
        L.scn_net_named.argtypes = [ctypes.c_char_p, c_int, c_int, c_int, c_f, c_int, c_int, c_int, c_f, c_int]
        L.scn_net_n_layers.argtypes = [c_p]
        L.scn_net_input_spatial_size.argtypes = [c_p]
        L.scn_net_layer_info.argtypes = [c_p, c_int, c_p, c_p]
        L.scn_net_set_weights.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.scn_net_load_weights.argtypes = [c_p, ctypes.c_char_p, c_int]
        L.scn_net_save_weights.argtypes = [c_p, ctypes.c_char_p, c_int]
        L.scn_net_set_precision.argtypes = [c_p, c_int]
        L.scn_net_forward_host.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p, c_p]
        L.scn_net_forward_device.argtypes = [c_p, c_int, c_int, c_int, c_p, c_p, c_p, c_p, c_p, c_p]
        L.scn_net_copy_probs_device.argtypes = [c_p, c_p]
        L.scn_net_train_batch.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p, c_f, c_f, c_p, c_p]
        L.scn_net_get_weights.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.scn_net_iface_dfeatures.restype, L.scn_net_iface_dfeatures.argtypes = c_ll, [c_p, c_int, c_p]
        L.scn_net_iface_sizes.argtypes = [c_p, c_int, c_p]
        L.scn_net_iface_fetch.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p]
        L.scn_net_take_multiply_adds.restype = c_d
        L.scn_net_enable_timing.argtypes = [c_p, c_int]
        L.scn_net_layer_times.argtypes = [c_p, c_p]
        L.scn_net_process_dataset.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p, c_int, c_p, c_p]
        L.scn_host_vectorTopIndices.argtypes = [c_p, c_int, c_int, c_p]
        L.scn_net_exchange_create.argtypes = [c_p, c_int, c_int, c_int, c_p]
        L.scn_net_exchange_buffer.restype, L.scn_net_exchange_buffer.argtypes = c_p, [c_p]
        L.scn_net_exchange_connect.argtypes = [c_p, c_p]
        L.scn_net_exchange_connect_local.argtypes = [c_p, c_p]
        L.scn_net_exchange_destroy.argtypes = [c_p]
        L.scn_net_forward_host_exchange.argtypes = [c_p, c_int] + [c_p] * 7
        L.scn_net_exchange_flush.argtypes = [c_p, c_p, c_p]
        L.scn_net_exchange_step_device.argtypes = [c_p, c_p, c_int, c_p, c_p]
        L.scn_net_forward_host_begin.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.scn_net_rescale_batch.argtypes = [c_p, c_int, c_p, c_p, c_p]
        L.scn_net_set_dropout_features.argtypes = [c_p, c_int, c_p, c_int]
        L.scn_net_addIndexLearnerLayer.argtypes = [c_p]
        L.scn_net_index_learner_batch.argtypes = [c_p, c_int, c_p, c_p, c_p, c_p, c_f, c_f, c_p, c_p]
        L.scn_net_iface_present.argtypes = [c_p, c_int, c_p]
        L.scn_net_forward_host_end.argtypes = [c_p, c_p, c_p, c_p, c_p]
        _lib = L
    return _lib


def _np(a):
    return None if a is None else a.ctypes.data_as(c_p)


def _check(rc):
    if rc != 0:
        raise abi.ScnError(lib().scn_net_last_error().decode())


class Net:
    """A SparseConvNetCUDA.  lattice 0 = SparseConvNet (square/cubic), 1 = SparseConvTriangLeNet.
    Kernels are enqueued on torch's current stream at construction time."""

    def __init__(self, dim, nInputFeatures, nClasses, nTop=1, lattice=0, handle=None, own_stream=False):
        self.L = lib()
        self.dim, self.nIn, self.nClasses, self.nTop, self.lattice = dim, nInputFeatures, nClasses, nTop, lattice
        if handle is None:
            stream = None if own_stream else _current_stream()
            handle = self.L.scn_net_create(dim, nInputFeatures, nClasses, nTop, lattice, stream)
            if not handle:
                raise abi.ScnError(self.L.scn_net_last_error().decode())
        self.h = c_p(handle)

    @classmethod
    def DeepCNet(cls, dim, l, k, fn, nInputFeatures, nClasses, p=0.0, nTop=1):
        L = lib()
        h = L.scn_net_DeepCNet(dim, l, k, fn, nInputFeatures, nClasses, p, nTop, _current_stream())
        if not h:
            raise abi.ScnError(L.scn_net_last_error().decode())
        return cls(dim, nInputFeatures, nClasses, nTop, 0, handle=h)

    @classmethod
    def named(cls, name, dim, l, k, fn, nInputFeatures, nClasses, p=0.0, nTop=1, fmpShrink=0.0):
        """One of the named architectures of NetworkArchitectures.h, constructed through its class; the
        network runs on a stream of its own, as the reference's does."""
        L = lib()
        h = L.scn_net_named(name.encode(), dim, l, k, fmpShrink, fn, nInputFeatures, nClasses, p, nTop)
        if not h:
            raise abi.ScnError(L.scn_net_last_error().decode())
        return cls(dim, nInputFeatures, nClasses, nTop, 0, handle=h)

    def close(self):
        if self.h:
            self.L.scn_net_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def addLeNetLayerMP(self, nFeatures, fs, fstride, ps, pstride, act=abi.RELU, dropout=0.0, minActive=1):
        _check(self.L.scn_net_addLeNetLayerMP(self.h, nFeatures, fs, fstride, ps, pstride, act, dropout, minActive))

    def addLeNetLayerFMP(self, kind, nFeatures, fs, fstride, ps, fmpShrink, act=abi.RELU, dropout=0.0, minActive=1):
        """Convolution block + fractional max-pooling: kind FMP_PO, FMP_PD, FMP_RO or FMP_RD."""
        _check(self.L.scn_net_addLeNetLayerFMP(self.h, kind, nFeatures, fs, fstride, ps, fmpShrink, act, dropout, minActive))

    def set_pool_fusion(self, on):
        """Fuse convolution + learnt layer + non-overlapping max pooling into one kernel (default) or not."""
        _check(self.L.scn_net_set_pool_fusion(self.h, int(bool(on))))

    def seed_fmp(self, seed):
        """Re-seed every FMP layer's RNG (layer l gets seed + l) before the next forward."""
        _check(self.L.scn_net_seed_fmp(self.h, seed))

    def addTerminalPoolingLayer(self, poolSize):
        _check(self.L.scn_net_addTerminalPoolingLayer(self.h, poolSize))

    def addSoftmaxLayer(self):
        _check(self.L.scn_net_addSoftmaxLayer(self.h))

    @property
    def inputSpatialSize(self):
        return self.L.scn_net_input_spatial_size(self.h)

    def layers(self):
        out = []
        for i in range(self.L.scn_net_n_layers(self.h)):
            info = np.zeros(10, np.int32)
            d = c_f()
            _check(self.L.scn_net_layer_info(self.h, i, _np(info), ctypes.byref(d)))
            rec = dict(zip(LAYER_KEYS, (int(v) for v in info)))
            rec["dropout"] = float(d.value)
            out.append(rec)
        return out

    def set_weights(self, i, W, B, prelu=None):
        W = np.ascontiguousarray(W, np.float32)
        B = np.ascontiguousarray(B, np.float32)
        prelu = None if prelu is None else np.ascontiguousarray(prelu, np.float32)
        _check(self.L.scn_net_set_weights(self.h, i, _np(W), _np(B), _np(prelu)))

    def load_weights(self, base, epoch):
        _check(self.L.scn_net_load_weights(self.h, base.encode(), epoch))

    def save_weights(self, base, epoch):
        _check(self.L.scn_net_save_weights(self.h, base.encode(), epoch))

    def set_precision(self, precision):
        _check(self.L.scn_net_set_precision(self.h, precision))

    def forward_host(self, keys, off, features):
        """numpy in (int32 keys with -1 for background rows, int32 offsets, float32 features),
        numpy out: (probabilities, predictions)."""
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        B = len(off) - 1
        probs = np.empty((B, self.nClasses), np.float32)
        pred = np.empty((B, self.nTop), np.int32)
        _check(self.L.scn_net_forward_host(self.h, B, _np(keys), _np(off), _np(features), _np(probs), _np(pred)))
        return probs, pred

    def forward_host_begin(self, keys, off, features):
        """Starts the upload of a batch (int32 keys, int32 offsets, float32 features: contiguous arrays that the caller
        keeps alive and unchanged until the matching forward_host_end); at most two batches may be on their way."""
        for a, t in ((keys, np.int32), (off, np.int32), (features, np.float32)):
            if a.dtype != t or not a.flags["C_CONTIGUOUS"]:
                raise abi.ScnError("forward_host_begin takes contiguous int32 / int32 / float32 arrays (no copies are made)")
        B = len(off) - 1
        _check(self.L.scn_net_forward_host_begin(self.h, B, _np(keys), _np(off), _np(features)))
        self._begun = getattr(self, "_begun", []) + [(B, keys, off, features)]

    def forward_host_end(self, exchange=False, gathered_prev=None, rows_prev=None):
        """Computes the oldest batch begun; returns (probs, pred) or, with exchange, (probs, pred, gathered_prev, rows_prev)."""
        if not getattr(self, "_begun", None):
            raise abi.ScnError("no batch is on its way (forward_host_begin)")
        B = self._begun.pop(0)[0]
        probs = np.empty((B, self.nClasses), np.float32)
        pred = np.empty((B, self.nTop), np.int32)
        if exchange:
            world, cap = self._exchange
            if gathered_prev is None:
                gathered_prev = np.empty((world, cap, self.nClasses), np.float32)
            if rows_prev is None:
                rows_prev = np.empty(world, np.int32)
        _check(self.L.scn_net_forward_host_end(self.h, _np(probs), _np(pred), _np(gathered_prev) if exchange else None,
                                               _np(rows_prev) if exchange else None))
        return (probs, pred, gathered_prev, rows_prev) if exchange else (probs, pred)

    # ---- results of a batch sharded over the GPUs of one node (peer stores, no host-side collective)
    def exchange_create(self, world, rank, cap_rows):
        """Allocates this rank's exchange buffer; returns the 64 bytes the other ranks need (bytes)."""
        h = (ctypes.c_ubyte * 64)()
        _check(self.L.scn_net_exchange_create(self.h, world, rank, cap_rows, h))
        self._exchange = (world, cap_rows)
        return bytes(h)

    def exchange_buffer(self):
        return self.L.scn_net_exchange_buffer(self.h)

    def exchange_connect(self, handles):
        """handles: the ranks' 64-byte entries in rank order (bytes of length world * 64)."""
        buf = (ctypes.c_ubyte * len(handles)).from_buffer_copy(handles)
        _check(self.L.scn_net_exchange_connect(self.h, buf))

    def exchange_connect_local(self, buffers):
        """buffers: every rank's exchange_buffer() pointer, for ranks that live in this process."""
        arr = (c_p * len(buffers))(*buffers)
        _check(self.L.scn_net_exchange_connect_local(self.h, arr))

    def exchange_destroy(self):
        _check(self.L.scn_net_exchange_destroy(self.h))

    def forward_host_exchange(self, keys, off, features, gathered_prev=None, rows_prev=None):
        """forward_host that also publishes this step's probabilities to every rank; returns (probs, pred,
        gathered_prev[world, cap_rows, nClasses], rows_prev[world]): what every rank published in the step before
        (rows_prev all -1 on the first step)."""
        world, cap = self._exchange
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        B = len(off) - 1
        probs = np.empty((B, self.nClasses), np.float32)
        pred = np.empty((B, self.nTop), np.int32)
        if gathered_prev is None:
            gathered_prev = np.empty((world, cap, self.nClasses), np.float32)
        if rows_prev is None:
            rows_prev = np.empty(world, np.int32)
        _check(self.L.scn_net_forward_host_exchange(self.h, B, _np(keys), _np(off), _np(features), _np(probs), _np(pred),
                                                    _np(gathered_prev), _np(rows_prev)))
        return probs, pred, gathered_prev, rows_prev

    def exchange_flush(self, gathered=None, rows=None):
        """The blocks of the last published step (waits for the stream)."""
        world, cap = self._exchange
        if gathered is None:
            gathered = np.empty((world, cap, self.nClasses), np.float32)
        if rows is None:
            rows = np.empty(world, np.int32)
        _check(self.L.scn_net_exchange_flush(self.h, _np(gathered), _np(rows)))
        return gathered, rows

    def exchange_step_device(self, d_probs, rows, d_gathered_prev, d_rows_status_prev):
        """Enqueue: collect the step before into the two device tensors, then publish d_probs (None: collect only)."""
        _check(self.L.scn_net_exchange_step_device(self.h, None if d_probs is None else c_p(d_probs.data_ptr()), rows,
                                                   c_p(d_gathered_prev.data_ptr()), c_p(d_rows_status_prev.data_ptr())))

    def forward_device(self, d_keys, d_off, d_bg, d_features, max_sites, d_probs=None, d_top=None):
        """torch CUDA tensors in and out; returns (d_probs, d_top) without synchronising."""
        B = d_bg.numel()
        rows = d_keys.numel()
        if d_probs is None:
            d_probs = torch.empty((B, self.nClasses), dtype=torch.float32, device=d_keys.device)
        if d_top is None:
            d_top = torch.empty((B, self.nTop), dtype=torch.int32, device=d_keys.device)
        _check(self.L.scn_net_forward_device(self.h, B, rows, int(max_sites), c_p(d_keys.data_ptr()), c_p(d_off.data_ptr()),
                                             c_p(d_bg.data_ptr()), c_p(d_features.data_ptr()), c_p(d_probs.data_ptr()),
                                             c_p(d_top.data_ptr())))
        return d_probs, d_top

    def train_batch(self, keys, off, features, labels, learning_rate, momentum):
        """One training step (forward, classifier, backward with SGD updates) -> (probabilities, dict(nll, mistakes))."""
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        labels = np.ascontiguousarray(labels, np.int32)
        B = len(off) - 1
        probs = np.empty((B, self.nClasses), np.float32)
        stats = np.zeros(2, np.float64)
        _check(self.L.scn_net_train_batch(self.h, B, _np(keys), _np(off), _np(features), _np(labels), learning_rate, momentum, _np(probs), _np(stats)))
        return probs, dict(nll=float(stats[0]), mistakes=int(stats[1]))

    def addIndexLearnerLayer(self):
        _check(self.L.scn_net_addIndexLearnerLayer(self.h))

    def index_learner_batch(self, keys, off, features, sample_numbers, learning_rate, momentum):
        """One index-learning step: every picture is its own class among the pictures of the batch.
        -> (probabilities [batch x batch], dict(nll, mistakes))."""
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        sample_numbers = np.ascontiguousarray(sample_numbers, np.int32)
        B = len(off) - 1
        probs = np.zeros((B, B), np.float32)
        stats = np.zeros(2, np.float64)
        _check(self.L.scn_net_index_learner_batch(self.h, B, _np(keys), _np(off), _np(features), _np(sample_numbers), learning_rate, momentum,
                                                  _np(probs), _np(stats)))
        return probs, dict(nll=float(stats[0]), mistakes=int(stats[1]))

    def rescale_batch(self, keys, off, features):
        """One RESCALEBATCH: every learnt layer's weights are rescaled from the statistics of its output on this batch."""
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        _check(self.L.scn_net_rescale_batch(self.h, len(off) - 1, _np(keys), _np(off), _np(features)))

    def set_dropout_features(self, layer, present):
        """The output features learnt layer `layer` keeps in the training batches that follow (ascending indices; an empty
        list returns to random draws)."""
        present = np.ascontiguousarray(present, np.int32)
        _check(self.L.scn_net_set_dropout_features(self.h, layer, _np(present), len(present)))

    def iface_present(self, i):
        """The features interface i kept in the last batch (all of them outside training with dropout)."""
        n = self.L.scn_net_iface_present(self.h, i, None)
        if n < 0:
            raise abi.ScnError(self.L.scn_net_last_error().decode())
        out = np.zeros(n, np.int32)
        if n:
            self.L.scn_net_iface_present(self.h, i, _np(out))
        return out

    def get_weights(self, i):
        L = self.layers()[i]
        W, B = np.zeros((L["nIn"], L["nOut"]), np.float32), np.zeros(L["nOut"], np.float32)
        pr = np.zeros(L["nOut"], np.float32)
        _check(self.L.scn_net_get_weights(self.h, i, _np(W), _np(B), _np(pr)))
        return W, B, (pr if L["act"] == abi.PRELU else None)

    def dfeatures(self, i):
        n = self.L.scn_net_iface_dfeatures(self.h, i, None)
        if n < 0:
            raise abi.ScnError(self.L.scn_net_last_error().decode())
        d = np.zeros(n, np.float32)
        if n:
            self.L.scn_net_iface_dfeatures(self.h, i, _np(d))
        return d

    def copy_probs_device(self, d_probs):
        _check(self.L.scn_net_copy_probs_device(self.h, c_p(d_probs.data_ptr())))
        return d_probs

    def iface(self, i, features=True):
        s = np.zeros(5, np.int64)
        _check(self.L.scn_net_iface_sizes(self.h, i, _np(s)))
        rows, nF, sp, nr, nc = (int(v) for v in s)
        feat = np.zeros((rows, nF), np.float32) if features else None
        rules = np.zeros(nr, np.int32)
        ch = np.zeros(nc, np.int32) if nc else None
        rk = np.zeros(rows, np.int32)
        _check(self.L.scn_net_iface_fetch(self.h, i, _np(feat), _np(rules), _np(ch), _np(rk)))
        return dict(nSpatialSites=rows, nFeatures=nF, spatialSize=sp, features=feat, rules=rules,
                    choices=ch if ch is not None else np.zeros(0, np.int32), row_keys=rk)

    def enable_timing(self, on=True):
        _check(self.L.scn_net_enable_timing(self.h, int(on)))

    def layer_times(self):
        n = self.L.scn_net_n_layers(self.h)
        ms = np.zeros(n + 1, np.float32)
        _check(self.L.scn_net_layer_times(self.h, _np(ms)))
        return ms

    def process_dataset(self, keys, off, features, labels, batch_size):
        keys = np.ascontiguousarray(keys, np.int32)
        off = np.ascontiguousarray(off, np.int32)
        features = np.ascontiguousarray(features, np.float32)
        labels = None if labels is None else np.ascontiguousarray(labels, np.int32)
        n = len(off) - 1
        probs = np.empty((n, self.nClasses), np.float32)
        err = c_f()
        _check(self.L.scn_net_process_dataset(self.h, n, _np(keys), _np(off), _np(features), _np(labels), batch_size,
                                              ctypes.byref(err), _np(probs)))
        return float(err.value), probs


def take_multiply_adds():
    return lib().scn_net_take_multiply_adds()


def host_top_indices(v, k):
    v = np.ascontiguousarray(v, np.float32)
    out = np.zeros(k, np.int32)
    _check(lib().scn_host_vectorTopIndices(_np(v), len(v), k, _np(out)))
    return out
