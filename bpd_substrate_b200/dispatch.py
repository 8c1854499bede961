"""Host side of the quantized decode dispatch.

Mirrors the GEMV schedule of the reference's GPU decode driver
(inference/llamatov_gpu_llama.py:119-166): per layer seven weight-times-vector products
(q, k, v, o, gate, up, down), called through the C ABI.  Where the reference dequantizes every
tensor to fp32 on the CPU and uploads ``[K, N]`` floats (``:64-74``), this keeps the Q4_K
bytes on the device (0.5625 B per weight instead of 4) and runs ``gpu_vecmat_q4k``-style
kernels on them.

Everything here goes through ``libbpdq.so`` (ctypes); there is no CPU path.

A :class:`LayerSet` owns one contiguous device arena for the activations of a whole step and
one for its outputs, so that a step's inputs arrive with one host-to-device copy and its
results leave with one device-to-host copy.
"""
import ctypes as C

import numpy as np

from . import capi, synth

GROUPS_DECODE = ((0, 1, 2), (3,), (4, 5), (6,))       # q/k/v share x, gate/up share x
GROUPS_NONE = ((0,), (1,), (2,), (3,), (4,), (5,), (6,))


class LayerSet:
    """``n_layers`` copies of a decoder layer's seven Q4_K matrices, resident on the device.

    shapes: sequence of (name, rows, cols).  The GEMVs of a step are independent of each other
    (each has its own activation vector), as in the benchmark configuration; ``schedule``
    chooses how they are launched:

    * ``"separate"`` -- one launch per matrix (the reference's call sequence);
    * ``"grouped"``  -- matrices that read the same vector in a real decoder (q/k/v, gate/up)
      share a launch and the first member's activation vector;
    * ``"batched"``  -- the seven independent products of a layer go to the device as ONE
      launch (``bpd_qmatmul_q4k_q8k_batch_cuda``), each with its own activation vector.
    """

    def __init__(self, shapes=synth.MISTRAL_LAYER, n_layers=32, seed=2000, row_shard=(0, 1), lib=None,
                 d_out=None, tokens=1):
        self.lib = lib or capi.load()
        self.shapes = tuple(shapes)
        self.n_layers = n_layers
        self.tokens = tokens       # activation rows per product (1 = decode; more: schedule "separate" only)
        rank, world = row_shard
        self.rank, self.world = rank, world
        lib = self.lib
        rng = np.random.default_rng(seed + 7919 * rank)
        # rows of every matrix are split evenly over the ranks (contiguous row ranges)
        self.local = []
        for name, rows, cols in self.shapes:
            assert rows % world == 0, f"{name}: {rows} rows do not divide over {world} ranks"
            self.local.append((name, rows // world, cols))
        self.x_off, self.o_off = [], []
        xo = oo = 0
        for _ in range(n_layers):
            for _, rows, cols in self.local:
                self.x_off.append(xo)
                self.o_off.append(oo)
                xo += tokens * cols * 4
                oo += tokens * rows * 4
        self.x_bytes, self.o_bytes = xo, oo
        self.d_x = lib.bpdq_alloc(xo)
        self._own_out = d_out is None      # an output arena may be lent by the caller (e.g. for NCCL)
        self.d_out = lib.bpdq_alloc(oo) if d_out is None else d_out
        self.weights = []          # [layer][matrix] device pointers
        self.weight_bytes = 0
        base = [synth.q4k_matrix(rows, cols, rng) for _, rows, cols in self.local]
        for layer in range(n_layers):
            ptrs = []
            for m, (_, rows, cols) in enumerate(self.local):
                # every layer gets its own bytes (same distribution): rotate by whole super-blocks
                w = np.roll(base[m], synth.Q4K_BYTES * (layer + 1))
                p = lib.bpdq_alloc(w.nbytes)
                lib.bpdq_h2d(p, w.ctypes.data, w.nbytes)
                ptrs.append(p)
                self.weight_bytes += w.nbytes
            self.weights.append(ptrs)
        self.base_weights = base   # host copy of layer "-1" (layer l = roll by l+1 blocks)
        self.stream = lib.bpdq_stream_create()
        self.graph = {}
        self._keep = []
        self.ws = None             # scratch for quantized activations (batched schedule)
        capi.check(lib.bpdq_last_status(), "LayerSet setup")

    # ---- sizes
    def algorithmic_bytes(self):
        """Quantized weights + fp32 activations in + fp32 outputs out, per step."""
        return self.n_layers * sum(synth.gemv_bytes_q4k(rows, cols, self.tokens) for _, rows, cols in self.local)

    def launches_per_step(self, schedule):
        if self.tokens > 1:
            return 2 * self.n_layers * len(self.local)   # activation quantizer + GEMM kernel per matrix
        if schedule == "batched":
            return 2 * self.n_layers      # activation quantizer + GEMV kernel per layer
        return self.n_layers * len(GROUPS_DECODE if schedule == "grouped" else GROUPS_NONE)

    def host_weight(self, layer, m):
        return np.roll(self.base_weights[m], synth.Q4K_BYTES * (layer + 1))

    # ---- launches
    def _group_args(self, layer, members):
        idx = [layer * len(self.local) + m for m in members]
        n = len(members)
        wp = (C.c_void_p * n)(*[self.weights[layer][m] for m in members])
        op = (C.c_void_p * n)(*[self.d_out + self.o_off[i] for i in idx])
        mp = (C.c_int * n)(*[self.local[m][1] for m in members])
        self._keep.append((wp, op, mp))
        return n, wp, op, mp, self.d_x + self.x_off[idx[0]], self.local[members[0]][2]

    def enqueue_step(self, schedule="grouped", stream=None):
        """Queues one decode step's GEMVs on ``stream`` (default: this object's stream)."""
        lib, s = self.lib, (stream if stream is not None else self.stream)
        if self.tokens > 1:
            # several tokens per product: one launch per matrix (tensor-core kernel above 4 tokens)
            nm = len(self.local)
            for layer in range(self.n_layers):
                for m, (_, rows, cols) in enumerate(self.local):
                    i = layer * nm + m
                    capi.check(lib.bpd_qmm_q4k_q8k_cuda(self.weights[layer][m], self.d_x + self.x_off[i],
                                                        self.d_out + self.o_off[i], self.tokens, rows, cols, 0, 0,
                                                        None, s), "GEMM launch")
            return
        if schedule == "batched":
            nm = len(self.local)
            for layer in range(self.n_layers):
                descs = (capi.GemvDesc * nm)()
                for m, (_, rows, cols) in enumerate(self.local):
                    i = layer * nm + m
                    descs[m] = capi.GemvDesc(self.weights[layer][m], self.d_x + self.x_off[i],
                                             self.d_out + self.o_off[i], rows, cols)
                if self.ws is None:
                    self.ws_stride = (lib.bpdq_batch_workspace_bytes(nm, descs) + 255) // 256 * 256
                    self.ws = lib.bpdq_alloc(self.ws_stride * self.n_layers)
                # every layer has its own scratch: launches of one step never share it
                capi.check(lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(nm, descs, self.ws + layer * self.ws_stride,
                                                                 self.ws_stride, s), "batched GEMV launch")
            return
        groups = GROUPS_DECODE if schedule == "grouped" else GROUPS_NONE
        for layer in range(self.n_layers):
            for members in groups:
                if len(members) == 1:
                    i = layer * len(self.local) + members[0]
                    _, rows, cols = self.local[members[0]]
                    rc = lib.bpd_qmatmul_q4k_q8k_cuda(self.weights[layer][members[0]], self.d_x + self.x_off[i],
                                                      self.d_out + self.o_off[i], rows, cols, s)
                else:
                    n, wp, op, mp, x, K = self._group_args(layer, members)
                    rc = lib.bpd_qmatmul_q4k_q8k_multi_cuda(n, wp, op, mp, x, K, s)
                capi.check(rc, "GEMV launch")

    def capture(self, schedule="grouped"):
        """Records a step into a CUDA graph (launch gaps disappear, PDL edges are kept)."""
        if schedule not in self.graph:
            lib = self.lib
            self.enqueue_step(schedule)              # warm-up outside capture (attributes, caches)
            capi.check(lib.bpdq_stream_sync(self.stream))
            capi.check(lib.bpdq_graph_begin(self.stream), "graph capture")
            self.enqueue_step(schedule)
            g = lib.bpdq_graph_end(self.stream)
            if not g:
                raise capi.BpdqError(f"graph capture failed (status {lib.bpdq_last_status()})")
            self.graph[schedule] = g
        return self.graph[schedule]

    def step(self, schedule="grouped"):
        """One step with inputs already on the device (asynchronous on self.stream)."""
        capi.check(self.lib.bpdq_graph_launch(self.capture(schedule), self.stream), "graph launch")

    def step_host(self, x_host_ptr, out_host_ptr, schedule="grouped"):
        """One step from HOST buffers: copies the step's activations in, runs it, copies the
        outputs back and waits.  Pointers should be pinned (bpdq_host_alloc)."""
        lib = self.lib
        capi.check(lib.bpdq_h2d_async(self.d_x, x_host_ptr, self.x_bytes, self.stream))
        self.step(schedule)
        capi.check(lib.bpdq_d2h_async(out_host_ptr, self.d_out, self.o_bytes, self.stream))
        capi.check(lib.bpdq_stream_sync(self.stream))

    # ---- data movement helpers
    def upload_activations(self, x_all):
        x_all = np.ascontiguousarray(x_all, dtype=np.float32)
        assert x_all.nbytes == self.x_bytes
        self.lib.bpdq_h2d(self.d_x, x_all.ctypes.data, self.x_bytes)

    def download_outputs(self):
        out = np.empty(self.o_bytes // 4, np.float32)
        self.lib.bpdq_stream_sync(self.stream)
        self.lib.bpdq_d2h(out.ctypes.data, self.d_out, self.o_bytes)
        return out

    def activation_slice(self, x_all, layer, m):
        i = layer * len(self.local) + m
        return x_all[self.x_off[i] // 4: self.x_off[i] // 4 + self.local[m][2]]

    def output_slice(self, out_all, layer, m):
        i = layer * len(self.local) + m
        return out_all[self.o_off[i] // 4: self.o_off[i] // 4 + self.local[m][1]]

    def close(self):
        lib = self.lib
        lib.bpdq_stream_sync(self.stream)
        for g in self.graph.values():
            lib.bpdq_graph_destroy(g)
        self.graph = {}
        for ptrs in self.weights:
            for p in ptrs:
                lib.bpdq_free(p)
        self.weights = []
        lib.bpdq_free(self.d_x)
        if self.ws is not None:
            lib.bpdq_free(self.ws)
        if self._own_out:
            lib.bpdq_free(self.d_out)
        lib.bpdq_stream_destroy(self.stream)
