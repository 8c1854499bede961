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
      launch (``bpd_qmatmul_q4k_q8k_batch_cuda``), each with its own activation vector;
    * ``"persistent"`` -- the products of the step (or of a range of its layers) as persistent launches of up
      to 128 products each, whose weight ring never drains between layers (``bpdq_gemv_stream_run_ready``),
      each after one launch that quantizes its vectors.
    """

    def __init__(self, shapes=synth.MISTRAL_LAYER, n_layers=32, seed=2000, row_shard=(0, 1), lib=None,
                 d_out=None, tokens=1, retile=None):
        self.lib = lib or capi.load()
        self.shapes = tuple(shapes)
        self.n_layers = n_layers
        self.tokens = tokens       # activation rows per product (1 = decode)
        # several activation rows per product: the weights are held re-tiled in groups of 16 rows (one copy, the
        # permutation of bpd_repack_q4k_rg16_cuda) and the step runs as persistent launches of the MMA kernel on them
        self.retiled = (tokens > 1) if retile is None else bool(retile)
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
                if self.retiled:
                    t = lib.bpdq_alloc(lib.bpd_q4k_rg16_bytes(rows, cols))
                    capi.check(lib.bpd_repack_q4k_rg16_cuda(p, t, rows, cols, None), "bpd_repack_q4k_rg16_cuda")
                    lib.bpdq_sync()
                    lib.bpdq_free(p)
                    p = t
                ptrs.append(p)
                self.weight_bytes += w.nbytes
            self.weights.append(ptrs)
        self.base_weights = base   # host copy of layer "-1" (layer l = roll by l+1 blocks)
        self.stream = lib.bpdq_stream_create()
        self.graph = {}
        self._keep = []
        self.ws = None             # scratch for quantized activations (batched schedule)
        self.stream_plans = {}     # (first, last) -> (plan, scratch) of the persistent schedule
        self.copy_streams = self.copy_events = None   # second and third stream of step_host
        self.even_ranges = False                      # True: step_host's ranges of layers all the same size
        capi.check(lib.bpdq_last_status(), "LayerSet setup")

    # ---- sizes
    def multi_token_kernel(self, schedule):
        """Name of the kernel that does the work when every product has several activation rows."""
        if self.retiled:
            return "k_gemm_q4k_rg16"
        return "k_gemm_q4k_q8k_mma / k_gemm_q4k_q8k_tc5 / k_gemv_q4k_q8k (one launch per matrix, by token count and size)"

    def algorithmic_bytes(self):
        """Quantized weights + fp32 activations in + fp32 outputs out, per step."""
        return self.n_layers * sum(synth.gemv_bytes_q4k(rows, cols, self.tokens) for _, rows, cols in self.local)

    def launches_per_step(self, schedule):
        if self.retiled:
            return self.lib.bpdq_gemm_rg16_stream_launches(self._stream_plan(0, self.n_layers)[0])
        if self.tokens > 1:
            return 2 * self.n_layers * len(self.local)   # activation quantizer + GEMM kernel per matrix
        if schedule == "persistent":
            # quantizer + persistent GEMV kernel per 128 products
            return self.lib.bpdq_gemv_stream_launches(self._stream_plan(0, self.n_layers)[0])
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

    def enqueue_step(self, schedule="grouped", stream=None, layers=None, tag=None):
        """Queues one decode step's GEMVs on ``stream`` (default: this object's stream); ``layers`` =
        (first, last+1) restricts it to a range of layers."""
        lib, s = self.lib, (stream if stream is not None else self.stream)
        first, last = layers if layers is not None else (0, self.n_layers)
        if self.retiled:
            capi.check(lib.bpdq_gemm_rg16_stream_run(self._stream_plan(first, last, tag)[0], s), "persistent GEMM launch")
            return
        if self.tokens > 1:
            # several tokens per product on the original rows: one launch per matrix (tensor-core kernel above 4 tokens)
            nm = len(self.local)
            for layer in range(first, last):
                for m, (_, rows, cols) in enumerate(self.local):
                    i = layer * nm + m
                    capi.check(lib.bpd_qmm_q4k_q8k_cuda(self.weights[layer][m], self.d_x + self.x_off[i],
                                                        self.d_out + self.o_off[i], self.tokens, rows, cols, 0, 0,
                                                        None, s), "GEMM launch")
            return
        if schedule == "persistent":
            # the step's activations are all on the device before its first launch (independent products): the
            # quantizer may read them ahead of stream order
            capi.check(lib.bpdq_gemv_stream_run_ready(self._stream_plan(first, last, tag)[0], s), "persistent GEMV launch")
            return
        if schedule == "batched":
            nm = len(self.local)
            for layer in range(first, last):
                descs = (capi.GemvDesc * nm)()
                for m, (_, rows, cols) in enumerate(self.local):
                    i = layer * nm + m
                    descs[m] = capi.GemvDesc(self.weights[layer][m], self.d_x + self.x_off[i],
                                             self.d_out + self.o_off[i], rows, cols)
                if self.ws is None:
                    self.ws_stride = (lib.bpdq_batch_workspace_bytes(nm, descs) + 255) // 256 * 256
                    self.ws = lib.bpdq_alloc(self.ws_stride * self.n_layers)
                # every layer has its own scratch and the step's activations are all on the device before
                # its first launch (independent products): the quantizers may run ahead of stream order
                capi.check(lib.bpd_qmatmul_q4k_q8k_batch_ready_cuda(nm, descs, self.ws + layer * self.ws_stride,
                                                                    self.ws_stride, s), "batched GEMV launch")
            return
        groups = GROUPS_DECODE if schedule == "grouped" else GROUPS_NONE
        for layer in range(first, last):
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

    def _stream_plan(self, first, last, tag=None):
        """Plan (and record scratch) of the persistent schedule for layers [first, last); made on first use.  Peer
        targets registered at that moment are part of the plan, so plans made under different registrations carry
        different tags."""
        key = (first, last, tag)
        if key not in self.stream_plans:
            lib, nm = self.lib, len(self.local)
            descs = (capi.GemvDesc * (nm * (last - first)))()
            for layer in range(first, last):
                for m, (_, rows, cols) in enumerate(self.local):
                    i = layer * nm + m
                    descs[i - first * nm] = capi.GemvDesc(self.weights[layer][m], self.d_x + self.x_off[i],
                                                          self.d_out + self.o_off[i], rows, cols)
            if self.retiled:
                ws_bytes = lib.bpdq_gemm_rg16_stream_workspace_bytes(len(descs), descs, self.tokens)
                ws = lib.bpdq_alloc(ws_bytes)
                plan = lib.bpdq_gemm_rg16_stream_create(len(descs), descs, self.tokens, ws, ws_bytes)
            else:
                ws_bytes = lib.bpdq_batch_workspace_bytes(len(descs), descs)
                ws = lib.bpdq_alloc(ws_bytes)
                plan = lib.bpdq_gemv_stream_create(len(descs), descs, ws, ws_bytes)
            if not plan:
                lib.bpdq_free(ws)
                raise capi.BpdqError(f"stream plan rejected (status {lib.bpdq_last_status()})")
            self.stream_plans[key] = (plan, ws)
        return self.stream_plans[key]

    def drop_stream_plans(self):
        """Forgets the persistent schedule's plans (they are rebuilt on next use, e.g. after the peer targets changed)."""
        self.lib.bpdq_stream_sync(self.stream)
        for plan, ws in self.stream_plans.values():
            (self.lib.bpdq_gemm_rg16_stream_destroy if self.retiled else self.lib.bpdq_gemv_stream_destroy)(plan)
            self.lib.bpdq_free(ws)
        self.stream_plans = {}

    def capture(self, schedule="grouped", layers=None, tag=None):
        """Records a step (or a range of its layers) into a CUDA graph (launch gaps disappear, PDL
        edges are kept).  tag: tells apart recordings of the same step made under different library
        state (the peer-store targets registered with bpdq_set_peer_outputs are read at recording time)."""
        key = schedule if layers is None else (schedule, tuple(layers))
        if tag is not None:
            key = (key, "tag", tag)
        if key not in self.graph:
            lib = self.lib
            self.enqueue_step(schedule, layers=layers, tag=tag)     # warm-up outside capture (attributes, caches)
            capi.check(lib.bpdq_stream_sync(self.stream))
            capi.check(lib.bpdq_graph_begin(self.stream), "graph capture")
            self.enqueue_step(schedule, layers=layers, tag=tag)
            g = lib.bpdq_graph_end(self.stream)
            if not g:
                raise capi.BpdqError(f"graph capture failed (status {lib.bpdq_last_status()})")
            self.graph[key] = g
        return self.graph[key]

    def step(self, schedule="grouped", layers=None, tag=None):
        """One step (or a range of its layers) with inputs already on the device (asynchronous on
        self.stream)."""
        capi.check(self.lib.bpdq_graph_launch(self.capture(schedule, layers, tag), self.stream), "graph launch")

    def layer_output_range(self, first, last):
        """(byte offset, bytes) of the outputs of layers [first, last) in the output arena."""
        nm = len(self.local)
        begin = self.o_off[first * nm]
        end = self.o_off[last * nm] if last < self.n_layers else self.o_bytes
        return begin, end - begin

    def step_host(self, x_host_ptr, out_host_ptr, schedule="grouped", chunks=4, tag=None, after=None):
        """One step from HOST buffers (pinned: bpdq_host_alloc): activations in, GEMVs, outputs back, wait.

        The step is cut into ``chunks`` ranges of layers; the activations of a range are copied in on a
        second stream and its outputs copied back on a third while other ranges compute, so that only
        the first range's copy-in and the last range's copy-out are not hidden.  ``chunks=1`` runs copy,
        step, copy in sequence on one stream.  ``tag``: which recording of the step to replay (see capture);
        ``after``: called when all launches are queued on self.stream and before the wait, e.g. to queue the
        flag exchange of a row-sharded step."""
        lib = self.lib
        n = max(1, min(chunks, self.n_layers))
        if n == 1:
            capi.check(lib.bpdq_h2d_async(self.d_x, x_host_ptr, self.x_bytes, self.stream))
            self.step(schedule, tag=tag)
            if after is not None:
                after()
            capi.check(lib.bpdq_d2h_async(out_host_ptr, self.d_out, self.o_bytes, self.stream))
            capi.check(lib.bpdq_stream_sync(self.stream))
            return
        if self.copy_streams is None:
            self.copy_streams = (lib.bpdq_stream_create(), lib.bpdq_stream_create())
            self.copy_events = [(lib.bpdq_event_create(), lib.bpdq_event_create()) for _ in range(self.n_layers)]
        s_in, s_out = self.copy_streams
        ranges = self.host_ranges(chunks)
        for c, (first, last) in enumerate(ranges):
            begin, nbytes = self.layer_input_range(first, last)
            capi.check(lib.bpdq_h2d_async(self.d_x + begin, x_host_ptr + begin, nbytes, s_in))
            capi.check(lib.bpdq_event_record(self.copy_events[c][0], s_in))
        for c, (first, last) in enumerate(ranges):
            capi.check(lib.bpdq_stream_wait_event(self.stream, self.copy_events[c][0]))
            self.step(schedule, (first, last), tag)
            capi.check(lib.bpdq_event_record(self.copy_events[c][1], self.stream))
            capi.check(lib.bpdq_stream_wait_event(s_out, self.copy_events[c][1]))
            begin, nbytes = self.layer_output_range(first, last)
            capi.check(lib.bpdq_d2h_async(out_host_ptr + begin, self.d_out + begin, nbytes, s_out))
        if after is not None:
            after()
        capi.check(lib.bpdq_stream_sync(s_out))
        capi.check(lib.bpdq_stream_sync(self.stream))

    def host_ranges(self, chunks):
        """The ranges of layers that step_host(chunks=...) runs as separate recordings."""
        n = max(1, min(chunks, self.n_layers))
        if n == 1:
            return [None]
        # Only the first range's copy-in and the last range's copy-out cannot hide behind other ranges' GEMVs, so
        # the ranges taper towards both ends (1 : 2 : 4 ... 4 : 2 : 1) when there are layers enough for that.
        taper = [min(1 << c, 1 << (n - 1 - c), 4) for c in range(n)] if self.n_layers >= 2 * n and not self.even_ranges else [1] * n
        total, acc, bounds = sum(taper), 0, [0]
        for c in range(n):
            acc += taper[c]
            bounds.append(max(bounds[-1] + 1, min(self.n_layers - (n - 1 - c), round(self.n_layers * acc / total))))
        bounds[-1] = self.n_layers
        return [(bounds[c], bounds[c + 1]) for c in range(n)]

    def layer_input_range(self, first, last):
        """(byte offset, bytes) of the activations of layers [first, last) in the input arena."""
        nm = len(self.local)
        begin = self.x_off[first * nm]
        end = self.x_off[last * nm] if last < self.n_layers else self.x_bytes
        return begin, end - begin

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
        return x_all[self.x_off[i] // 4: self.x_off[i] // 4 + self.tokens * self.local[m][2]]

    def output_slice(self, out_all, layer, m):
        i = layer * len(self.local) + m
        return out_all[self.o_off[i] // 4: self.o_off[i] // 4 + self.tokens * self.local[m][1]]

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
        if self.copy_streams is not None:
            for st in self.copy_streams:
                lib.bpdq_stream_destroy(st)
            for a, b in self.copy_events:
                lib.bpdq_event_destroy(a)
                lib.bpdq_event_destroy(b)
            self.copy_streams = None
        self.drop_stream_plans()
        if self.ws is not None:
            lib.bpdq_free(self.ws)
        if self._own_out:
            lib.bpdq_free(self.d_out)
        lib.bpdq_stream_destroy(self.stream)


class DecodeChain:
    """One token through ``n_layers`` decoder layers, in the order of the reference's decode loop
    (inference/llamatov_gpu_llama.py:119-166), as a DEPENDENT chain: every product reads what the
    step before it wrote.  As in that loop, attention over a single position is the identity and
    ``wo`` is applied to ``q`` directly (``:133-146``).

    Per layer the reference makes 13 launches (rms_norm, q, k, v, o, add, rms_norm, gate, silu,
    up, mul, down, add) on fp32 weights.  Modes here, all on Q4_K weights and all giving the same bits:

    * ``"chain"`` -- 8 launches: each elementwise step is a small kernel that writes the next
      product's activation records (``bpd_rmsnorm_q8k_records_cuda`` and friends), products that
      share an input share a launch, the residual add is the product's epilogue::

          rms_norm -> rec | q,k,v | q -> rec | o, += x | rms_norm -> rec | gate,up | silu(gate)*up -> rec | down, += x

    * ``"chain4"`` -- 4 launches: the step runs inside the product kernel that consumes it
      (``bpd_qmatmul_q4k_fused_cuda``), in every CTA.  Fewer launches, but 148 CTAs repeat the step
      after the wait for the previous launch: measured slower than ``"chain"`` on the benchmark's shapes;
    * ``"chain-separate"`` -- the reference's call sequence (gpu_rms_norm, gpu_silu, gpu_mul,
      gpu_add and one product per matrix);
    * ``"chain-persistent"`` -- ONE cooperative launch per token (plus the memset of its barrier
      counters): the 4-phase program of ``"chain4"`` for all layers inside one kernel whose warps refill
      their own rings across the phases, so the weights of the next phase are on their way during the barrier
      between phases; gate and up rows travel in pairs and the activation is formed where they meet
      (``bpdq_chain_run``).
    """

    MODES = {"chain": 8, "chain4": 4, "chain-separate": 13, "chain-persistent": 0}

    NAMES = ("wq", "wk", "wv", "wo", "w1", "w3", "w2")

    def __init__(self, hidden=4096, kv=1024, ffn=14336, n_layers=32, seed=3000, eps=1e-5, lib=None):
        self.lib = lib = lib or capi.load()
        self.hidden, self.kv, self.ffn, self.n_layers, self.eps = hidden, kv, ffn, n_layers, eps
        self.shapes = (("wq", hidden, hidden), ("wk", kv, hidden), ("wv", kv, hidden), ("wo", hidden, hidden),
                       ("w1", ffn, hidden), ("w3", ffn, hidden), ("w2", hidden, ffn))
        rng = np.random.default_rng(seed)
        self.base_weights = [synth.q4k_matrix(rows, cols, rng) for _, rows, cols in self.shapes]
        self.norm_host = (1.0 + 0.1 * rng.standard_normal((n_layers, 2, hidden))).astype(np.float32)
        self.weights, self.weight_bytes = [], 0
        for layer in range(n_layers):
            ptrs = []
            for m in range(7):
                w = self.host_weight(layer, m)
                p = lib.bpdq_alloc(w.nbytes)
                lib.bpdq_h2d(p, w.ctypes.data, w.nbytes)
                ptrs.append(p)
                self.weight_bytes += w.nbytes
            self.weights.append(ptrs)
        self.d_norm = lib.bpdq_alloc(self.norm_host.nbytes)
        lib.bpdq_h2d(self.d_norm, self.norm_host.ctypes.data, self.norm_host.nbytes)
        f = 4
        self.buf = {name: lib.bpdq_alloc(n * f) for name, n in
                    (("x", hidden), ("h", hidden), ("q", hidden), ("k", kv), ("v", kv), ("gate", ffn), ("up", ffn),
                     ("attn", hidden), ("down", hidden))}
        self.rec = {name: lib.bpdq_alloc(lib.bpdq_records_bytes(n)) for name, n in
                    (("h", hidden), ("q", hidden), ("act", ffn))}
        self.ws = lib.bpdq_alloc(lib.bpdq_records_bytes(ffn) + 4096)   # scratch of the separate (unfused) products
        self.ws_bytes = lib.bpdq_records_bytes(ffn) + 4096
        self.stream = lib.bpdq_stream_create()
        self.graph = {}
        self.program = None        # handle of the persistent-chain program, built on first use
        capi.check(lib.bpdq_last_status(), "DecodeChain setup")

    def host_weight(self, layer, m):
        return np.roll(self.base_weights[m], synth.Q4K_BYTES * (layer + 1))

    def norm_ptr(self, layer, which):
        return self.d_norm + (layer * 2 + which) * self.hidden * 4

    def algorithmic_bytes(self):
        """Quantized weights + fp32 vector in + fp32 vector out of every product, per token."""
        return self.n_layers * sum(synth.gemv_bytes_q4k(rows, cols) for _, rows, cols in self.shapes)

    @staticmethod
    def _mode(mode):
        if isinstance(mode, str):
            return mode
        return "chain" if mode else "chain-separate"

    def launches_per_token(self, mode="chain"):
        mode = self._mode(mode)
        return 1 if mode == "chain-persistent" else self.n_layers * self.MODES[mode]

    # ---- state
    def set_state(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        assert x.size == self.hidden
        self.lib.bpdq_h2d(self.buf["x"], x.ctypes.data, x.nbytes)

    def get_state(self):
        out = np.empty(self.hidden, np.float32)
        self.lib.bpdq_stream_sync(self.stream)
        self.lib.bpdq_d2h(out.ctypes.data, self.buf["x"], out.nbytes)
        return out

    # ---- launches
    def _descs(self, layer, members, outs):
        d = (capi.GemvDesc * len(members))()
        for j, (m, o) in enumerate(zip(members, outs)):
            _, rows, cols = self.shapes[m]
            d[j] = capi.GemvDesc(self.weights[layer][m], None, self.buf[o], rows, cols)
        return d

    def enqueue_token(self, mode="chain", stream=None):
        lib, s, b, r = self.lib, (stream if stream is not None else self.stream), self.buf, self.rec
        H, F, eps = self.hidden, self.ffn, self.eps
        mode = self._mode(mode)
        if mode == "chain-persistent":
            if self.program is None:
                ph = (capi.ChainPhase * (4 * self.n_layers))()
                for layer in range(self.n_layers):
                    for k, (members, outs, pro, a, bb, mask) in enumerate((
                            ((0, 1, 2), ("q", "k", "v"), 1, b["x"], self.norm_ptr(layer, 0), 0),
                            ((3,), ("x",), 0, b["q"], None, 1),
                            ((4, 5), ("gate", "up"), 1, b["x"], self.norm_ptr(layer, 1), 0),
                            ((6,), ("x",), 2, b["gate"], b["up"], 1))):
                        p = ph[4 * layer + k]
                        p.n, p.prologue, p.a, p.b, p.eps, p.accumulate_mask = len(members), pro, a, bb, eps, mask
                        for j, d in enumerate(self._descs(layer, members, outs)):
                            p.prod[j] = d
                self.program = lib.bpdq_chain_create(len(ph), ph)
                if not self.program:
                    raise capi.BpdqError(f"chain program rejected (status {lib.bpdq_last_status()})")
            capi.check(lib.bpdq_chain_run(self.program, s), "persistent chain launch")
            return
        if mode == "chain4":
            for layer in range(self.n_layers):
                capi.check(lib.bpd_qmatmul_q4k_fused_cuda(3, self._descs(layer, (0, 1, 2), ("q", "k", "v")), 1, b["x"],
                                                          self.norm_ptr(layer, 0), eps, 0, s))
                capi.check(lib.bpd_qmatmul_q4k_fused_cuda(1, self._descs(layer, (3,), ("x",)), 0, b["q"], None, 0.0, 1, s))
                capi.check(lib.bpd_qmatmul_q4k_fused_cuda(2, self._descs(layer, (4, 5), ("gate", "up")), 1, b["x"],
                                                          self.norm_ptr(layer, 1), eps, 0, s))
                capi.check(lib.bpd_qmatmul_q4k_fused_cuda(1, self._descs(layer, (6,), ("x",)), 2, b["gate"], b["up"], 0.0,
                                                          1, s))
            return
        if mode == "chain":
            for layer in range(self.n_layers):
                capi.check(lib.bpd_rmsnorm_q8k_records_cuda(b["x"], self.norm_ptr(layer, 0), r["h"], 1, H, eps, s))
                capi.check(lib.bpd_qmatmul_q4k_records_cuda(3, self._descs(layer, (0, 1, 2), ("q", "k", "v")), r["h"], 0, s))
                capi.check(lib.bpd_quant_q8k_records_cuda(b["q"], r["q"], H, s))
                capi.check(lib.bpd_qmatmul_q4k_records_cuda(1, self._descs(layer, (3,), ("x",)), r["q"], 1, s))
                capi.check(lib.bpd_rmsnorm_q8k_records_cuda(b["x"], self.norm_ptr(layer, 1), r["h"], 1, H, eps, s))
                capi.check(lib.bpd_qmatmul_q4k_records_cuda(2, self._descs(layer, (4, 5), ("gate", "up")), r["h"], 0, s))
                capi.check(lib.bpd_swiglu_q8k_records_cuda(b["gate"], b["up"], r["act"], F, s))
                capi.check(lib.bpd_qmatmul_q4k_records_cuda(1, self._descs(layer, (6,), ("x",)), r["act"], 1, s))
            return
        # the reference's call sequence; the fp32 ops launch on the library's current stream
        prev = lib.bpdq_get_stream()
        lib.bpdq_set_stream(s)

        def product(layer, m, x, out):
            _, rows, cols = self.shapes[m]
            d = (capi.GemvDesc * 1)(capi.GemvDesc(self.weights[layer][m], b[x], b[out], rows, cols))
            capi.check(lib.bpd_qmatmul_q4k_q8k_batch_ws_cuda(1, d, self.ws, self.ws_bytes, s))

        try:
            for layer in range(self.n_layers):
                lib.gpu_rms_norm(b["x"], self.norm_ptr(layer, 0), b["h"], 1, H, eps)
                product(layer, 0, "h", "q")
                product(layer, 1, "h", "k")
                product(layer, 2, "h", "v")
                product(layer, 3, "q", "attn")
                lib.gpu_add(b["x"], b["attn"], b["x"], H)
                lib.gpu_rms_norm(b["x"], self.norm_ptr(layer, 1), b["h"], 1, H, eps)
                product(layer, 4, "h", "gate")
                lib.gpu_silu(b["gate"], b["gate"], F)
                product(layer, 5, "h", "up")
                lib.gpu_mul(b["gate"], b["up"], b["gate"], F)
                product(layer, 6, "gate", "down")
                lib.gpu_add(b["x"], b["down"], b["x"], H)
            capi.check(lib.bpdq_last_status(), "decode chain")
        finally:
            lib.bpdq_set_stream(prev)

    def capture(self, mode="chain"):
        """Records one token's chain into a CUDA graph."""
        mode = self._mode(mode)
        if mode not in self.graph:
            lib = self.lib
            self.enqueue_token(mode)                 # warm-up outside capture (attributes, caches)
            capi.check(lib.bpdq_stream_sync(self.stream))
            capi.check(lib.bpdq_graph_begin(self.stream), "graph capture")
            self.enqueue_token(mode)
            g = lib.bpdq_graph_end(self.stream)
            if not g:
                raise capi.BpdqError(f"graph capture failed (status {lib.bpdq_last_status()})")
            self.graph[mode] = g
        return self.graph[mode]

    def step(self, mode="chain"):
        capi.check(self.lib.bpdq_graph_launch(self.capture(mode), self.stream), "graph launch")

    # ---- the part of LayerSet's interface that the benchmark driver uses (schedule = mode)
    @property
    def x_bytes(self):
        return self.hidden * 4

    o_bytes = x_bytes

    def launches_per_step(self, schedule):
        return self.launches_per_token(schedule)

    def upload_activations(self, x):
        self.set_state(x)

    def step_host(self, x_host_ptr, out_host_ptr, schedule="chain"):
        """One token from HOST buffers: hidden state in, chain, hidden state out, wait."""
        lib = self.lib
        capi.check(lib.bpdq_h2d_async(self.buf["x"], x_host_ptr, self.x_bytes, self.stream))
        self.step(schedule)
        capi.check(lib.bpdq_d2h_async(out_host_ptr, self.buf["x"], self.o_bytes, self.stream))
        capi.check(lib.bpdq_stream_sync(self.stream))

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
        if self.program:
            lib.bpdq_chain_destroy(self.program)
            self.program = None
        for p in list(self.buf.values()) + list(self.rec.values()) + [self.d_norm, self.ws]:
            lib.bpdq_free(p)
        lib.bpdq_stream_destroy(self.stream)
