"""The B200 sparse-attention backend: a drop-in for the reference's
``HybridSparseBackend`` (attention/sparse/backend.py:27-255) behind the same
duck-typed protocol the forward boundary calls
(attention_forward.py:99-128,148-246):

    prepare(q, k, v, *, layer_index, transformer_options) -> prepared
    prepare_projected(projected, *, layer_index, transformer_options) -> prepared
    execute(prepared) -> HND tensor (1,H,S,128) in the input dtype

``prepare`` runs, on torch's current stream and without a host sync:
column statistics (K mean, V amax) -> INT8 Q/K blocks with FP64 tile means ->
FP8 V carrier -> router.  ``execute`` launches the tcgen05 attention kernel.
There is no fallback of any kind: a device that is not sm_100, a missing
native library or a failed launch raises ``SparseSageError``.

Every wait inside the attention kernel is bounded; a wait that runs out makes
the kernel return early and leave a code in a per-device status word that the
backend hands to every launch.  Reading that word needs the stream to have
drained, so it is not done on the hot path: ``check_status()`` reads it (and
raises) whenever the caller synchronises anyway, ``forward_host`` calls it
before it returns, and the next ``prepare`` on the device looks at the word
through a pinned mirror filled by an asynchronous copy queued after the
previous launch, without blocking.
"""

from __future__ import annotations

import torch

from . import _native, ops
from .carriers import PreparedFusedQKV, PreparedHybrid, PreparedSparse, validate_prepared_fused_qkv
from .config import MODE_SAGE128_FUSED_QKV, HybridSparseConfig, resolve_video_budget
from .errors import FusedQKVError, SparseRouterError, SparseSageError
from .router import KV_TILE, Q_TILE, SparseTileRouter
from .runtime import get_runtime_snapshot

V_QUANT_BOUND = 448.0  # FP32 accumulation (reference: sparse_sage.py:296)


def preflight():
    """Raise ``SparseSageError`` unless the native library loads and the
    current device is sm_100 (reference: sparse_sage.py:261-310)."""
    if not torch.cuda.is_available():
        raise SparseSageError("Hybrid Sparse Attention requires CUDA")
    try:
        capability = ops.device_capability()
    except _native.NativeError as exc:
        raise SparseSageError("B200 sparse backend is unavailable: %s" % exc) from exc
    if capability // 10 != 10:
        raise SparseSageError("B200 sparse backend requires sm_100; device is sm_%d" % capability)
    return capability


class CapturedLayerCall:
    """``prepare`` + ``execute`` of one layer call on fixed input tensors, captured
    once into a CUDA graph.  A sampler calls the same layer with the same shapes
    and the same budget step after step; replaying the graph takes the host out
    of the step (about ten launches and a dozen stream operations otherwise) and
    closes the gaps between the small carrier kernels.  Every kernel still runs on
    every replay - statistics, carriers, router, attention (and, for a sharded
    owner, the exchange) - on whatever ``q``, ``k``, ``v`` hold at that moment; the
    output tensor and the carriers are the same buffers each time.  The device
    status word is not looked at between replays: call ``check_status()``.
    """

    def __init__(self, owner, q, k, v, *, layer_index, transformer_options, warmup=2):
        self.owner = owner
        # streams, status words, kernel attributes and exchange buffers come into being on the first
        # calls; none of that may happen inside the capture
        for _ in range(max(1, int(warmup))):
            owner.execute(owner.prepare(q, k, v, layer_index=layer_index, transformer_options=transformer_options))
        torch.cuda.synchronize(q.device)
        self.graph = torch.cuda.CUDAGraph()
        # thread-local error mode: a watchdog thread of a communication library may legally touch the
        # device while this thread captures
        with torch.cuda.graph(self.graph, capture_error_mode="thread_local"):
            self.prepared = owner.prepare(q, k, v, layer_index=layer_index, transformer_options=transformer_options)
            self.out = owner.execute(self.prepared)

    def replay(self):
        self.graph.replay()
        return self.out


class B200SparseBackend:
    name = "b200_sparse"
    requires_registered_sage = False
    requires_runtime_context = True
    approximate = True

    def __init__(self, config=None, *, router=None, projector=None, smooth_k=True, check_device=True):
        self.config = config or HybridSparseConfig()
        if not isinstance(self.config, HybridSparseConfig):
            raise TypeError("config must be HybridSparseConfig")
        if check_device:
            preflight()
        self.router = router if router is not None else SparseTileRouter(self.config)
        if (self.router.q_tile, self.router.kv_tile) != (Q_TILE, KV_TILE):
            raise SparseSageError(
                "router geometry %dQ x %dKV does not match the kernel's %dQ x %dKV"
                % (self.router.q_tile, self.router.kv_tile, Q_TILE, KV_TILE)
            )
        self.projector = projector
        if self.config.mode == MODE_SAGE128_FUSED_QKV and self.projector is None:
            from .projector import ChunkedSparseQKVProjector

            self.projector = ChunkedSparseQKVProjector()
        self.smooth_k = bool(smooth_k)
        self._status = {}  # device index -> (device int32[4], pinned mirror, event of the last mirror copy)

    # -- identity ---------------------------------------------------------

    @property
    def installation_signature(self):
        projector = self.projector
        return (
            self.name,
            self.config.signature,
            (type(self.router).__module__, type(self.router).__qualname__),
            ("sm_100a", Q_TILE, KV_TILE, "int8_qk", "fp8_e4m3_v", V_QUANT_BOUND, _native.ABI_VERSION),
            bool(self.smooth_k),
            None
            if projector is None
            else (
                type(projector).__module__,
                type(projector).__qualname__,
                getattr(projector, "name", None),
                getattr(projector, "installation_signature", None),
            ),
        )

    def as_status(self):
        return {
            "mode": self.config.mode,
            "video_budget": float(self.config.video_budget),
            "denser_early_late_steps": bool(self.config.denser_early_late_steps),
            "density_mode": self.config.density_mode,
            "sparge_attention": "h3sparse-abi-%d" % _native.ABI_VERSION,
            "sparse_architecture": "sm_100a",
            "sparse_q_tile": Q_TILE,
            "sparse_kv_tile": KV_TILE,
            "sparse_v_format": "fp8",
            "sparse_v_quant_bound": V_QUANT_BOUND,
            "sparse_extension_layout": "h3sparse",
            "approximate": True,
            "fused_qkv": self.projector is not None,
            "qkv_projector": getattr(self.projector, "name", None),
            "qkv_chunk_rows": getattr(self.projector, "chunk_rows", None),
            "smooth_k": bool(self.smooth_k),
        }

    # -- helpers ------------------------------------------------------------

    @staticmethod
    def _snapshot(transformer_options, sequence):
        snapshot = get_runtime_snapshot(transformer_options)
        if snapshot is None:
            raise SparseSageError("Sparse Attention requires an H3 runtime snapshot")
        if not snapshot.valid_layout:
            raise SparseSageError(
                "Sparse Attention requires a valid packed layout: %s"
                % (getattr(snapshot, "error", None) or "layout unavailable")
            )
        if int(snapshot.layout.seq_len) != int(sequence):
            raise SparseSageError(
                "runtime layout sequence %d does not match attention sequence %d"
                % (snapshot.layout.seq_len, sequence)
            )
        return snapshot

    @staticmethod
    def _metadata(mask_metadata, layer_index, heads):
        metadata = mask_metadata.as_dict()
        metadata.update(
            {
                "layer": int(layer_index),
                "sparse_sage_heads": int(heads),
                "total_q_video_tiles": int(mask_metadata.pure_video_q_tiles) * int(heads),
                "sparse_architecture": "sm_100a",
                "sparse_q_tile": Q_TILE,
                "sparse_kv_tile": KV_TILE,
                "sparse_v_format": "fp8",
                "sparse_accumulator": "f32",
                "sparse_v_quant_bound": V_QUANT_BOUND,
            }
        )
        return metadata

    @staticmethod
    def _sink(transformer_options, layer_index):
        recorder = (transformer_options or {}).get("h3_optimizations_attention_route")
        sink = getattr(recorder, "sink", None)
        return {} if sink is None else {"sink": sink(layer_index)}

    @staticmethod
    def _validate_qkv(q, k, v):
        if q.shape != k.shape or q.shape != v.shape:
            raise SparseSageError(
                "Sparse Sage requires equal self-attention Q/K/V shapes; got %s %s %s"
                % (tuple(q.shape), tuple(k.shape), tuple(v.shape))
            )
        if q.ndim != 4:
            raise SparseSageError("Sparse Sage expects HND rank-4 tensors")
        batch, heads, sequence, head_dim = q.shape
        if batch != 1:
            raise SparseSageError("released H3 expects attention batch 1; got %d" % batch)
        if head_dim != 128:
            raise SparseSageError("Sparse Sage requires head_dim 128; got %d" % head_dim)
        if q.dtype not in (torch.float16, torch.bfloat16, torch.float32) or q.dtype != k.dtype or q.dtype != v.dtype:
            raise SparseSageError("Sparse Sage Q/K/V require matching fp16, bf16 or fp32 dtypes")
        if q.device != k.device or q.device != v.device:
            raise SparseSageError("Sparse Sage Q/K/V devices differ")
        if any(t.stride(-1) != 1 for t in (q, k, v)):
            raise SparseSageError("Sparse Sage Q/K/V last dimension must be contiguous")
        if not q.is_cuda:
            raise SparseSageError("Sparse Sage requires CUDA")
        return heads, sequence

    def _side_stream(self, device):
        streams = self.__dict__.setdefault("_side_streams", {})
        key = device.index if device.index is not None else torch.cuda.current_device()
        if key not in streams:
            streams[key] = torch.cuda.Stream(device)
        return streams[key]

    # -- device status word -------------------------------------------------

    ABORT_NAMES = {1: "Q tile load", 2: "K/V tile load", 3: "free K/V stage", 4: "QK^T result", 5: "P from the softmax warps",
                   6: "free P buffer", 7: "P.V before a rescale", 8: "last P.V"}

    def _status_slot(self, device):
        key = device.index if device.index is not None else torch.cuda.current_device()
        slot = self._status.get(key)
        if slot is None:
            word = torch.zeros(4, dtype=torch.int32, device=device)
            mirror = torch.zeros(4, dtype=torch.int32).pin_memory()
            slot = self._status[key] = (word, mirror, torch.cuda.Event())
        return slot

    @classmethod
    def _raise_for(cls, words, where):
        code, cta, head, tile = (int(x) for x in words)
        if code != 0:
            raise SparseSageError(
                "Sparse attention kernel gave up waiting for %s (code %d) in CTA %d, head %d, query tile %d (%s); "
                "the output of that launch is invalid"
                % (cls.ABORT_NAMES.get(code, "an unknown event"), code, cta, head, tile, where))

    def _poll_status(self, device):
        """Non-blocking look at the mirror of the previous launch's status."""
        if torch.cuda.is_current_stream_capturing():
            return  # an event query is not allowed inside a capture; check_status() covers replays
        slot = self._status.get(device.index if device.index is not None else torch.cuda.current_device())
        if slot is not None and slot[2].query():
            self._raise_for(slot[1].tolist(), "reported by an earlier launch")

    def check_status(self, device=None):
        """Synchronise with the device and raise ``SparseSageError`` if a
        bounded device wait ran out in any attention launch since the last
        check.  Clears the word."""
        devices = list(self._status) if device is None else [torch.device(device).index]
        for key in devices:
            slot = self._status.get(key)
            if slot is None:
                continue
            words = slot[0].cpu().tolist()
            if words[0] != 0:
                slot[0].zero_()
                slot[1].zero_()
            self._raise_for(words, "found by check_status")

    # -- protocol -------------------------------------------------------------

    def prepare(self, q, k, v, *, layer_index, transformer_options):
        heads, sequence = self._validate_qkv(q, k, v)
        self._poll_status(q.device)
        snapshot = self._snapshot(transformer_options, sequence)
        video_budget = resolve_video_budget(
            self.config, snapshot.step_index, snapshot.total_steps, layer_index
        )
        try:
            geometry = self.router.geometry(snapshot.layout)
            retained = self.router._retained(video_budget, geometry)
            need_route = retained < geometry.pure_video_kv_tiles
            summary_dtype = torch.float64 if need_route else None
            # Two streams share the GPU.  The column statistics (K mean, V scale) run on a
            # second stream while the Q quantiser, which needs neither, starts at once on the
            # current one; the K quantiser joins when the statistics are in.  The V carrier
            # is held back until the K quantiser is through, so that this memory-bound
            # kernel runs beside the router, which is latency bound and leaves the memory
            # system idle, instead of sharing the bandwidth with the K quantiser.  Every
            # buffer is allocated on the current stream, which both chains rejoin before
            # returning.
            main = torch.cuda.current_stream(q.device)
            side = self._side_stream(q.device)
            k_mean, v_scale, scratch = ops.column_stats_buffers(heads, q.device, want_k_mean=self.smooth_k)
            v_carrier = ops.allocate_v_carrier(sequence, heads, v.device)
            events = self.__dict__.setdefault("_stats_events", {})
            pair = events.get(side)
            if pair is None:
                pair = events[side] = (torch.cuda.Event(), torch.cuda.Event())
            stats_done, k_done = pair
            side.wait_stream(main)
            try:
                with torch.cuda.stream(side):
                    ops.column_stats_into(k if self.smooth_k else None, v, k_mean, v_scale, scratch, V_QUANT_BOUND)
                    stats_done.record(side)
                q_int8, q_scale, q_summary = ops.quant_qk_blocks(q, Q_TILE, summary_dtype=summary_dtype)
                main.wait_event(stats_done)
                k_int8, k_scale, k_summary = ops.quant_qk_blocks(k, KV_TILE, mean=k_mean, summary_dtype=summary_dtype)
                if need_route:
                    k_done.record(main)
                with torch.cuda.stream(side):
                    if need_route:
                        side.wait_event(k_done)
                    ops.quant_v_fp8_into(v, v_scale, v_carrier, v_bound=V_QUANT_BOUND)
                if need_route:
                    route = self.router.build_route_from_summaries(
                        q_summary, k_summary, snapshot.layout, video_budget,
                        **self._sink(transformer_options, layer_index),
                    )
                else:
                    route = self.router.build_route(
                        q, k, snapshot.layout, video_budget, **self._sink(transformer_options, layer_index)
                    )
            finally:
                # on every exit path the main stream is ordered after the second one, so the
                # allocator cannot hand these buffers to someone else while it still runs
                main.wait_stream(side)
        except SparseRouterError as exc:
            raise SparseSageError("sparse routing failed: %s" % exc) from exc
        except _native.NativeError as exc:
            raise SparseSageError("carrier preparation failed: layer=%d: %s" % (layer_index, exc)) from exc
        sparse = PreparedSparse(
            q_int8=q_int8, k_int8=k_int8, v_carrier=v_carrier, q_scale=q_scale, k_scale=k_scale,
            v_scale=v_scale, route=route, output_dtype=q.dtype, output_shape=tuple(q.shape),
            layer_index=int(layer_index), sequence=int(sequence), heads=int(heads),
            metadata=self._metadata(route.metadata, layer_index, heads),
        )
        sparse.metadata["smooth_k"] = bool(self.smooth_k)
        return PreparedHybrid(sparse=sparse)

    def prepare_projected(self, projected, *, layer_index, transformer_options):
        try:
            validate_prepared_fused_qkv(projected)
        except FusedQKVError as exc:
            raise SparseSageError(str(exc)) from exc
        snapshot = self._snapshot(transformer_options, projected.sequence)
        video_budget = resolve_video_budget(
            self.config, snapshot.step_index, snapshot.total_steps, layer_index
        )
        heads, sequence = int(projected.heads), int(projected.sequence)
        if not projected.q_int8.is_cuda:
            raise SparseSageError("fused H3 Sparse Sage requires CUDA")
        try:
            route = self.router.build_route_from_summaries(
                projected.q_summary, projected.k_summary, snapshot.layout, video_budget,
                **self._sink(transformer_options, layer_index),
            )
            if projected.v_carrier is not None:
                v_carrier, v_scale = projected.v_carrier, projected.v_scale
            else:
                v_carrier, v_scale = ops.quant_v_fp8(projected.v, None, V_QUANT_BOUND)
        except SparseRouterError as exc:
            raise SparseSageError("sparse routing failed: %s" % exc) from exc
        except _native.NativeError as exc:
            raise SparseSageError("carrier preparation failed: layer=%d: %s" % (layer_index, exc)) from exc
        metadata = self._metadata(route.metadata, layer_index, heads)
        metadata.update(
            {
                "qkv_projection": "fused_int8",
                "smooth_k": bool(projected.smooth_k),
                "prepacked_fp8_v": projected.v_carrier is not None,
            }
        )
        sparse = PreparedSparse(
            q_int8=projected.q_int8, k_int8=projected.k_int8, v_carrier=v_carrier,
            q_scale=projected.q_scale, k_scale=projected.k_scale, v_scale=v_scale, route=route,
            output_dtype=projected.output_dtype, output_shape=(1, heads, sequence, projected.head_dim),
            layer_index=int(projected.layer_index), sequence=sequence, heads=heads, metadata=metadata,
        )
        return PreparedHybrid(sparse=sparse)

    def execute(self, prepared, out=None, peer_out_ptrs=None):
        """Run the attention kernel on prepared carriers.  ``out`` (optional) is
        an HND ``(1, H, S, 128)`` tensor or view to write into;
        ``peer_out_ptrs`` (head-sharded runs, see ``sharding.HeadShardedBackend``)
        are the device addresses of the same head slice inside the peers'
        outputs, which receive every tile as well."""
        sparse = prepared.sparse
        route = sparse.route
        geometry = route.geometry
        device = sparse.q_int8.device
        word, mirror, copied = self._status_slot(device)
        try:
            out_dtype = sparse.output_dtype
            result = ops.sparse_attention(
                sparse.q_int8, sparse.k_int8, sparse.v_carrier, sparse.q_scale, sparse.k_scale,
                sparse.v_scale, route.indices,
                q_start=geometry.pure_video_q_start, q_stop=geometry.pure_video_q_stop,
                out=out, out_dtype=out_dtype, status=word, peer_out_ptrs=peer_out_ptrs,
            )
            if not torch.cuda.is_current_stream_capturing():
                # (an event recorded inside a capture could not be queried afterwards: replays are
                # covered by check_status(), which reads the device word itself)
                mirror.copy_(word, non_blocking=True)  # 16 bytes, stream ordered behind the kernel
                copied.record(torch.cuda.current_stream(device))
            return result
        except _native.NativeError as exc:
            raise SparseSageError(
                "Sparse attention kernel failed: layer=%d sequence=%d heads=%d dtype=%s: %s"
                % (sparse.layer_index, sparse.sequence, sparse.heads, sparse.output_dtype, exc)
            ) from exc

    def capture(self, q, k, v, *, layer_index, transformer_options):
        """This layer call as a replayable CUDA graph (see ``CapturedLayerCall``)."""
        return CapturedLayerCall(self, q, k, v, layer_index=layer_index, transformer_options=transformer_options)

    def execute_projected(self, module, prepared):
        """Attention followed by the block's ``out_proj`` on the tensor cores:
        returns ``(S, hidden)`` as the forward boundary allows a backend to do
        (attention_forward.py:99-128; the reference's streamed backend does it in
        attention/sparse/sparse_sage_streamed.py:1454-1472).  The attention output
        is written token-major, so its ``(S, heads*128)`` view feeds the GEMM
        without a copy.  Returns ``None`` - the caller then runs ``execute`` and
        the module's own ``out_proj`` - when the projection is not a plain bf16
        Linear on the attention's device."""
        linear = getattr(module, "out_proj", None)
        weight = getattr(linear, "weight", None)
        sparse = prepared.sparse
        if (weight is None or weight.ndim != 2 or weight.dtype != torch.bfloat16
                or weight.dtype != sparse.output_dtype or weight.device != sparse.q_int8.device
                or weight.shape[1] != sparse.heads * 128 or weight.shape[0] % 8 or weight.stride(1) != 1):
            return None
        out_hnd = self.execute(prepared)                                   # (1, H, S, 128) view of (S, H, 128)
        rows = out_hnd.permute(0, 2, 1, 3).reshape(sparse.sequence, sparse.heads * 128)
        if rows.data_ptr() != out_hnd.data_ptr():                          # never a copy with this backend's buffers
            rows = rows.contiguous()
        bias = getattr(linear, "bias", None)
        try:
            result = ops.dense_gemm(rows, weight, bias=None if bias is None else bias.detach().float().contiguous())
        except _native.NativeError as exc:
            raise SparseSageError("output projection failed: layer=%d: %s" % (sparse.layer_index, exc)) from exc
        return result

    def forward(self, q, k, v, *, layer_index, transformer_options):
        """``prepare`` + ``execute`` for a batch: every sparse backend of the
        reference is limited to batch 1 (attention/sparse/sparse_sage.py:448-449)
        and so are ``prepare`` / ``execute`` here; batch elements are independent,
        so this entry walks them one after the other (one route per element) and
        returns ``(B, H, S, 128)``."""
        if q.ndim != 4 or q.shape != k.shape or q.shape != v.shape:
            raise SparseSageError("forward expects equal rank-4 HND Q/K/V; got %s %s %s"
                                  % (tuple(q.shape), tuple(k.shape), tuple(v.shape)))
        outputs = []
        for b in range(q.shape[0]):
            prepared = self.prepare(q[b:b + 1], k[b:b + 1], v[b:b + 1], layer_index=layer_index,
                                    transformer_options=transformer_options)
            outputs.append(self.execute(prepared))
        return outputs[0] if len(outputs) == 1 else torch.cat(outputs, dim=0)

    # -- host-resident activations -------------------------------------------

    def forward_host(self, q, k, v, out=None, *, layer_index, transformer_options, heads_per_chunk=None):
        """``prepare`` + ``execute`` for Q/K/V that live in (pinned) HOST memory.

        Heads are independent on the whole path, so the call walks the heads in
        chunks and overlaps three things on three streams: the host-to-device
        copy of chunk c+1, the kernels of chunk c (on the current stream) and
        the device-to-host copy of the output of chunk c-1.  The PCIe input copy
        is the longest of the three, so the call takes about as long as that
        copy alone.  Returns ``out`` (host, HND ``(1, H, S, 128)``; allocated
        pinned when not given).  With a route sink installed the heads are not
        split (the sink expects one call per layer).  The call returns once the
        output is in host memory and raises if a launch reported an expired
        device wait."""
        if q.is_cuda or k.is_cuda or v.is_cuda:
            raise SparseSageError("forward_host expects host tensors; use prepare/execute for device tensors")
        if q.shape != k.shape or q.shape != v.shape or q.ndim != 4 or q.shape[0] != 1 or q.shape[3] != 128:
            raise SparseSageError("forward_host expects equal (1, H, S, 128) Q/K/V; got %s %s %s"
                                  % (tuple(q.shape), tuple(k.shape), tuple(v.shape)))
        if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
            raise SparseSageError("forward_host expects contiguous HND host tensors")
        _, heads, sequence, _ = q.shape
        if out is None:
            out = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        elif out.shape != q.shape or out.dtype != q.dtype or out.is_cuda or not out.is_contiguous():
            raise SparseSageError("forward_host: out must be a contiguous host tensor shaped and typed like q")
        recorder = (transformer_options or {}).get("h3_optimizations_attention_route")
        whole = getattr(recorder, "sink", None) is not None
        if heads_per_chunk is None:
            # at least four chunks when the heads allow it, so that copy-in, kernels and copy-out overlap
            heads_per_chunk = 2 if heads >= 8 else 1
        chunk = heads if whole else max(1, min(int(heads_per_chunk), heads))
        bounds = [(a, min(a + chunk, heads)) for a in range(0, heads, chunk)]
        device = torch.device("cuda", torch.cuda.current_device())
        main = torch.cuda.current_stream(device)
        state = self._host_pipeline(device, chunk, sequence, q.dtype, min(3, len(bounds)))
        h2d, d2h, slots = state["h2d"], state["d2h"], state["slots"]
        h2d.wait_stream(main)
        d2h.wait_stream(main)
        for index, (a, b) in enumerate(bounds):
            slot = slots[index % len(slots)]
            n = b - a
            with torch.cuda.stream(h2d):
                if index >= len(slots):
                    h2d.wait_event(slot["computed"])  # the kernels of the chunk that used this slot are done
                for name, src in (("q", q), ("k", k), ("v", v)):
                    slot[name][:, :n].copy_(src[:, a:b], non_blocking=True)
                slot["loaded"].record(h2d)
            main.wait_event(slot["loaded"])
            if index >= len(slots):
                main.wait_event(slot["stored"])  # its previous output has left the device
            prepared = self.prepare(slot["q"][:, :n], slot["k"][:, :n], slot["v"][:, :n],
                                    layer_index=layer_index, transformer_options=transformer_options)
            self.execute(prepared, out=slot["out"][:, :n])
            slot["computed"].record(main)
            with torch.cuda.stream(d2h):
                d2h.wait_event(slot["computed"])
                out[:, a:b].copy_(slot["out"][:, :n], non_blocking=True)
                slot["stored"].record(d2h)
        main.wait_stream(d2h)
        main.wait_stream(h2d)
        main.synchronize()  # the result lives in host memory: it is complete when the call returns
        self.check_status(device)
        return out

    def _host_pipeline(self, device, chunk, sequence, dtype, n_slots):
        key = (device.index, int(chunk), int(sequence), dtype, int(n_slots))
        cache = self.__dict__.setdefault("_host_pipelines", {})
        state = cache.get(key)
        if state is None:
            cache.clear()  # one geometry at a time: the staging buffers are large
            shape = (1, chunk, sequence, 128)
            slots = []
            for _ in range(n_slots):
                slot = {name: torch.empty(shape, dtype=dtype, device=device) for name in ("q", "k", "v", "out")}
                slot.update({name: torch.cuda.Event() for name in ("loaded", "computed", "stored")})
                slots.append(slot)
            state = {"h2d": torch.cuda.Stream(device), "d2h": torch.cuda.Stream(device), "slots": slots}
            cache[key] = state
        return state

    def reference_lut(self, prepared):
        """The route in the reference's delta-LUT encoding ``(lut, valid)``."""
        sparse = prepared.sparse
        lut, valid, _ = self.router._lut(sparse.route, sparse.q_int8.device, sparse.heads)
        return lut, valid
