"""The kernel table of the product path: thin ctypes wrappers over `csrc/`.

Every method checks what its kernel cannot check (devices, dtypes, contiguity),
launches on torch's current stream and raises if the launch failed.  There is no
other implementation behind these calls: without a CUDA device or without the
compiled library, construction fails.
"""

from __future__ import annotations

import ctypes

import torch

from . import trace
from .build import build as _build_library

_F32, _BF16 = 0, 1
ERR_UNSUPPORTED = 10001


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _F32
    if t.dtype == torch.bfloat16:
        return _BF16
    raise TypeError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _check(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise KernelError("the kernels of this engine run on a CUDA device only; got a "
                              f"{t.device} tensor")
        if not t.is_contiguous():
            raise KernelError("kernel arguments must be contiguous")


class CudaOps:
    name = "cuda"

    def __init__(self) -> None:
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        major, minor = torch.cuda.get_device_capability()
        if major != 10:
            raise KernelError(f"the kernels are built for sm_100a; this device is sm_{major}{minor}")
        self.lib_path = _build_library()
        self.lib = ctypes.CDLL(self.lib_path)
        self.lib.somi_attention_generic_q_tile.restype = ctypes.c_int
        self.generic_q_tile = int(self.lib.somi_attention_generic_q_tile())
        self.lib.somi_prefill_q_tile.restype = ctypes.c_int
        self.prefill_q_tile = int(self.lib.somi_prefill_q_tile())
        self.lib.somi_prefill_tc_q_tile.restype = ctypes.c_int
        self.prefill_tc_q_tile = int(self.lib.somi_prefill_tc_q_tile())
        self.lib.somi_prefill_pp_q_tile.restype = ctypes.c_int
        self.prefill_pp_q_tile = int(self.lib.somi_prefill_pp_q_tile())
        self.lib.somi_latent_attention_generic_q_tile.restype = ctypes.c_int
        self.latent_q_tile = int(self.lib.somi_latent_attention_generic_q_tile())
        self.q_tile_sizes = tuple(dict.fromkeys((
            self.generic_q_tile, self.prefill_q_tile, self.prefill_tc_q_tile,
            self.prefill_pp_q_tile, self.latent_q_tile)))
        self.max_taps = int(self.lib.somi_causal_taps_max())
        self.use_mma_latent = True
        assert int(self.lib.somi_latent_attention_mma_q_tile()) == self.latent_q_tile
        self.use_pp_prefill = True
        self.pp_prefill_min_ctas = torch.cuda.get_device_properties(0).multi_processor_count
        self.use_tc_prefill = True
        self._q_maps: dict = {}
        self.lib.somi_decode_chunk.restype = ctypes.c_int
        self.decode_chunk = int(self.lib.somi_decode_chunk())
        self._workspace = None
        self._device_index = torch.cuda.current_device()
        self._tensor_maps: dict = {}
        self.use_tma_decode = True
        self.lib.somi_decode_ring_chunks.argtypes = [ctypes.c_int]
        self.lib.somi_decode_ring_chunks.restype = None
        self.use_tma_prefill = True
        self._gemm_maps: dict = {}
        self.use_skinny_gemm = True
        self.skinny_max_tokens = int(self.lib.somi_skinny_gemm_max_tokens())
        self._retired: list = []
        self.launches = 0     # kernels of this library launched so far

    # ------------------------------------------------------------------ util
    def _stream(self) -> ctypes.c_void_p:
        # the raw handle of the current stream, without the Python stream object in between:
        # that path costs microseconds per launch, which a step of hundreds of launches feels
        return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(self._device_index))

    def _done(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc == ERR_UNSUPPORTED:
            raise KernelError(f"{what}: these sizes are not supported by the kernel")
        if rc != 0:
            raise KernelError(f"{what}: CUDA error {rc}")

    def check_attention_geometry(self, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
        if head_dim % 16 or not 16 <= head_dim <= 256:
            raise KernelError(f"head_dim {head_dim} is not supported: the attention kernels take "
                              "multiples of 16 from 16 to 256")
        if num_kv_heads <= 0 or num_heads % num_kv_heads:
            raise KernelError(f"{num_heads} query heads cannot be grouped over {num_kv_heads} "
                              "key/value heads")

    # --------------------------------------------------------------- kernels
    def embed(self, ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
        _check(ids, table, out)
        assert ids.dtype == torch.int32 and out.dtype == torch.float32
        rc = self.lib.somi_embed(_ptr(ids), _ptr(table), _code(table), _ptr(out),
                                 ctypes.c_int(ids.shape[0]), ctypes.c_int(table.shape[1]),
                                 self._stream())
        self._done(rc, "embed")
        if trace.active():
            n = ids.shape[0] * table.shape[1]
            trace.note("embed", n * (table.element_size() + 4))

    def add_rmsnorm(self, residual, delta, weight, eps, out, rows=None) -> None:
        """residual += delta (float32, in place); out = rmsnorm(residual) * weight.

        `delta` is [N, H] in the compute dtype, or float32 [splits, N, H] partial sums that are
        added in order.  With `rows`, only those rows are produced and residual is not written.
        """
        _check(residual, delta, weight, out, rows)
        assert residual.dtype == torch.float32
        H = residual.shape[1]
        n_out = out.shape[0]
        splits, stride = 1, 0
        if delta is not None and delta.dim() == 3:
            assert delta.dtype == torch.float32
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        rc = self.lib.somi_add_rmsnorm(
            _ptr(residual), _ptr(delta), _code(delta) if delta is not None else _F32,
            ctypes.c_int(splits), ctypes.c_longlong(stride),
            _ptr(weight), _code(weight), ctypes.c_float(eps), _ptr(out), _code(out), _ptr(rows),
            ctypes.c_int(n_out), ctypes.c_int(H), ctypes.c_int(0 if rows is not None else 1),
            self._stream())
        self._done(rc, "add_rmsnorm")
        if trace.active():
            n = n_out * H
            moved = n * (4 + out.element_size()) + H * weight.element_size()
            if delta is not None:
                moved += splits * n * delta.element_size()
            if rows is None:
                moved += n * 4
            trace.note("add_rmsnorm", moved, detail=f"splits={splits}" if splits > 1 else "")

    def rope_store(self, qkv, positions, inv_freq, nq, nkv, hd, rotary_dim, slot_map, kcache,
                   vcache, partials=None, bias=None) -> None:
        """Rotate q and k of `qkv` in place and store k, v at their cache slots.

        With `partials` (float32 [splits, T, width], the output of a split-K projection) the
        projection is summed here, `bias` added, and `qkv` (bfloat16) only receives the queries.
        """
        _check(qkv, positions, inv_freq, slot_map, kcache, vcache, partials, bias)
        page_size = kcache.shape[2] if kcache is not None else 1
        if kcache is not None and slot_map is not None:
            assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
        if partials is not None:
            assert partials.dtype == torch.float32 and qkv.dtype == torch.bfloat16
            rc = self.lib.somi_rope_store_partial(
                _ptr(partials), ctypes.c_int(partials.shape[0]),
                ctypes.c_longlong(partials.shape[1] * partials.shape[2]), _ptr(bias),
                _code(bias) if bias is not None else _F32, _ptr(qkv), _ptr(positions),
                _ptr(inv_freq), ctypes.c_int(qkv.shape[0]), ctypes.c_int(nq), ctypes.c_int(nkv),
                ctypes.c_int(hd), ctypes.c_int(rotary_dim), _ptr(slot_map), _ptr(kcache),
                _ptr(vcache), ctypes.c_int(page_size), self._stream())
            self._done(rc, "rope_store_partial")
            if trace.active():
                n = qkv.shape[0] * qkv.shape[1]
                trace.note("rope_store", partials.shape[0] * n * 4 + n * 2, detail="from partial sums")
            return
        rc = self.lib.somi_rope_store(
            _ptr(qkv), _code(qkv), _ptr(positions), _ptr(inv_freq), ctypes.c_int(qkv.shape[0]),
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(rotary_dim),
            _ptr(slot_map), _ptr(kcache), _ptr(vcache), ctypes.c_int(page_size), self._stream())
        self._done(rc, "rope_store")
        if trace.active():
            n = qkv.shape[0] * qkv.shape[1]
            trace.note("rope_store", n * qkv.element_size() * 2)

    def _scratch(self, n_floats: int, device) -> torch.Tensor:
        """Float32 scratch that outlives the call (kernels of a captured graph keep its address)."""
        if self._workspace is None or self._workspace.numel() < n_floats:
            if self._workspace is not None:
                self._retired.append(self._workspace)
            self._workspace = torch.empty(max(n_floats, 1 << 20), dtype=torch.float32, device=device)
        return self._workspace

    def prefill_supported(self, nq: int, nkv: int, hd: int, dtype) -> bool:
        return dtype == torch.bfloat16 and bool(self.lib.somi_prefill_supported(
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd)))

    def decode_supported(self, nq: int, nkv: int, hd: int, dtype) -> bool:
        return dtype == torch.bfloat16 and bool(self.lib.somi_decode_supported(
            ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd)))

    def _kv_tensor_map(self, storage: torch.Tensor, hd: int, page_size: int):
        """A TMA tensor map over a cache group's whole storage, seen as [rows, hd] bfloat16."""
        key = (storage.data_ptr(), storage.numel(), hd, page_size)
        entry = self._tensor_maps.get(key)
        if entry is None:
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_kv_tensor_map(ctypes.c_void_p(addr), _ptr(storage),
                                                  ctypes.c_longlong(storage.numel() // hd),
                                                  ctypes.c_int(hd), ctypes.c_int(page_size))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over the cache (code {rc})")
            entry = (raw, addr)
            self._tensor_maps[key] = entry
        return entry[1]

    def set_decode_ring_chunks(self, chunks: int) -> None:
        """Chunks of 128 keys that one CTA of the TMA decode kernel walks through: 0 lets the
        launcher choose from the step's size (the default), 1 forces the one-chunk kernel,
        2..8 the ring kernel with that many."""
        self.lib.somi_decode_ring_chunks(int(chunks))

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for all kernels of the library (on by default)."""
        self.lib.somi_set_pdl(ctypes.c_int(1 if on else 0))

    def _q_tensor_map(self, qkv: torch.Tensor) -> int:
        key = (qkv.data_ptr(), qkv.shape[0], qkv.shape[1])
        entry = self._q_maps.get(key)
        if entry is None:
            if len(self._q_maps) > 4096:
                self._q_maps.clear()
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_q_tensor_map(ctypes.c_void_p(addr), _ptr(qkv),
                                                 ctypes.c_longlong(qkv.shape[0]),
                                                 ctypes.c_longlong(qkv.shape[1]))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over the projection buffer (code {rc})")
            entry = (raw, addr)
            self._q_maps[key] = entry
        return entry[1]

    def check_errors(self) -> None:
        """Raise if a kernel recorded that one of its bounded waits ran out (synchronises)."""
        if int(self.lib.somi_decode_tma_error()) != 0:
            raise KernelError("the TMA decode attention kernel gave up waiting for a copy; "
                              "its results are not valid")
        if int(self.lib.somi_prefill_tma_error()) != 0:
            raise KernelError("the TMA prefill attention kernel gave up waiting for a copy; "
                              "its results are not valid")
        if int(self.lib.somi_prefill_pp_error()) != 0:
            raise KernelError("the two-tile tcgen05 prefill attention kernel gave up waiting on a "
                              "barrier; its results are not valid")
        if int(self.lib.somi_prefill_tc_error()) != 0:
            raise KernelError("the tcgen05 prefill attention kernel gave up waiting on a barrier; "
                              "its results are not valid")
        if int(self.lib.somi_gemm_error()) != 0:
            raise KernelError("the tcgen05 matrix product gave up waiting on a barrier; "
                              "its results are not valid")

    @staticmethod
    def _attention_work(batch, first: int, last: int, nq: int, nkv: int, hd: int, elt: int,
                        window: int) -> tuple[float, float]:
        """Bytes and flops of attention for requests [first, last) of the batch: every key and
        value of a request's context once, queries in and outputs out; two products per
        (query, key) pair that the mask leaves."""
        moved = flops = 0.0
        cu, ctx = batch.host.cu_q, batch.host.ctx_len
        for r in range(first, last):
            q, c = int(cu[r + 1] - cu[r]), int(ctx[r])
            pairs = q * c + q * (q + 1) // 2
            kv = c + q
            if window < 0:         # a chunk of -window positions
                n = -window
                pairs = sum((c + i) % n + 1 for i in range(q)) if q < 4096 else min(pairs, q * n // 2)
                kv = min(kv, (c % n) + q)
            elif window:
                pairs = sum(min(c + i + 1, window) for i in range(q)) if q < 4096 else min(pairs, q * window)
                kv = min(kv, window + q - 1)
            moved += 2 * kv * nkv * hd * elt + 2 * q * nq * hd * elt
            flops += 4.0 * nq * hd * pairs
        return moved, flops

    def paged_attention(self, qkv, kcache, vcache, batch, group, nq, nkv, hd, scale, window,
                        out, storage=None, value_dim=None, chunk=None, gate=None,
                        gate_per_head=False, softcap=None, sinks=None) -> None:
        """Attention of every token of the step over the cache (keys/values already stored).

        In bfloat16 with head sizes 32/64/128, portions of prompts go to the tensor-core
        prefill kernel and single-token requests to the split-KV kernel (at most 16 query
        heads per kv head); float32 and every other size go to the generic kernel.  So do values
        of another width than the keys (`value_dim`) and a chunked mask (`chunk`: a token sees
        the earlier tokens of its own chunk of that many positions).  `gate`: logits [T, nq *
        value width] (rows may lie further apart); the output is multiplied by their sigmoid;
        with `gate_per_head` the logits are [T, nq], one per token and head.  `softcap`: scores
        pass cap * tanh(score / cap); `sinks`: float32 [nq] scores that join the softmax's
        denominator without a key.  With capped scores or sinks, bfloat16 prompt portions of head
        sizes 64/128 run the one-tile tcgen05 kernel (or the `mma.sync` kernel that TMA feeds) and
        single tokens the cp.async split-KV kernel; a per-head gate is then a kernel of its own
        behind them.
        """
        _check(qkv, kcache, vcache, out, group.block_table)
        assert kcache.dtype == qkv.dtype
        page_size = kcache.shape[2]
        win = int(window) if window else 0
        vd = int(value_dim) if value_dim else hd
        chunk = int(chunk) if chunk else 0
        if gate is not None and not (gate.is_cuda and gate.dtype == out.dtype and gate.stride(1) == 1
                                     and tuple(gate.shape) == ((out.shape[0], nq) if gate_per_head
                                                               else tuple(out.shape))):
            raise KernelError("an output gate is [T, heads * value width] (or [T, heads]) of the "
                              "output's dtype with contiguous rows")
        cap = float(softcap) if softcap else 0.0
        if sinks is not None:
            _check(sinks)
            assert sinks.dtype == torch.float32 and sinks.numel() == nq
        n_decode = batch.num_requests - batch.num_prefill_requests
        # what the tensor-core kernels compute; they fetch query rows in 16-byte pieces
        plain = vd == hd and qkv.shape[1] % 8 == 0
        shaped = cap != 0.0 or sinks is not None
        if chunk and win:
            raise KernelError("a mask is a window or a chunk, not both")
        split = plain and n_decode > 0 and self.decode_supported(nq, nkv, hd, qkv.dtype)
        tensor_core_prefill = (plain and batch.num_prefill_requests > 0
                               and self.prefill_supported(nq, nkv, hd, qkv.dtype))
        shaped_tc = False
        if shaped and tensor_core_prefill:
            # two kernels shape scores: the one-tile tcgen05 kernel and the TMA-fed mma.sync one
            geometry = (ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(page_size))
            shaped_tc = (self.use_tc_prefill and storage is not None
                         and bool(self.lib.somi_prefill_tc_supported(*geometry)))
            tensor_core_prefill = shaped_tc or (
                self.use_tma_prefill and storage is not None
                and bool(self.lib.somi_prefill_tma_supported(*geometry)))
        # the tensor-core kernels take the mask as one number: n > 0 a window, n < 0 a chunk of -n
        if chunk:
            win = -chunk
        if tensor_core_prefill:
            # Four kernels, the first that takes the sizes: both products on tcgen05 with
            # accumulators in tensor memory, two query tiles per CTA in ping-pong and the
            # probabilities handed on through tensor memory; the same with one query tile per CTA
            # and the probabilities through shared memory; mma.sync fed by TMA; mma.sync fed by
            # cp.async gathers.
            sizes = (ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(page_size))
            row_bytes = hd * 2
            # (the two-tile kernel has half as many CTAs: below one per SM the one-tile kernel,
            # with twice as many, is the faster: 0.5B shape at 2,048 tokens 123 vs 148 TFLOP/s)
            if shaped_tc:
                tiles = batch.tiles[self.prefill_tc_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tc_shaped(
                    ctypes.c_void_p(self._q_tensor_map(qkv)),
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), ctypes.c_float(cap), _ptr(sinks),
                    _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tc")
                kernel = "attention_prefill_tcgen05"
            elif shaped:
                tiles = batch.tiles[self.prefill_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tma_shaped(
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)), _ptr(qkv),
                    ctypes.c_int(qkv.shape[1]),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), ctypes.c_float(cap), _ptr(sinks),
                    _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tma")
                kernel = "attention_prefill_tma"
            elif (self.use_pp_prefill and storage is not None and qkv.shape[1] % 8 == 0
                    and batch.tiles[self.prefill_pp_q_tile].shape[0] * nq >= self.pp_prefill_min_ctas
                    and bool(self.lib.somi_prefill_pp_supported(*sizes))):
                tiles = batch.tiles[self.prefill_pp_q_tile]
                rc = self.lib.somi_paged_attention_prefill_pp(
                    ctypes.c_void_p(self._q_tensor_map(qkv)),
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_pp")
                kernel = "attention_prefill_tcgen05_pingpong"
            elif (self.use_tc_prefill and storage is not None and qkv.shape[1] % 8 == 0
                    and bool(self.lib.somi_prefill_tc_supported(*sizes))):
                tiles = batch.tiles[self.prefill_tc_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tc(
                    ctypes.c_void_p(self._q_tensor_map(qkv)),
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tc")
                kernel = "attention_prefill_tcgen05"
            elif (self.use_tma_prefill and storage is not None
                  and bool(self.lib.somi_prefill_tma_supported(*sizes))):
                tiles = batch.tiles[self.prefill_q_tile]
                rc = self.lib.somi_paged_attention_prefill_tma(
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)), _ptr(qkv),
                    ctypes.c_int(qkv.shape[1]),
                    ctypes.c_longlong((kcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    ctypes.c_longlong((vcache.data_ptr() - storage.data_ptr()) // row_bytes),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill_tma")
                kernel = "attention_prefill_tma"
            else:
                tiles = batch.tiles[self.prefill_q_tile]
                rc = self.lib.somi_paged_attention_prefill(
                    _ptr(qkv), ctypes.c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                    _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]), *sizes,
                    ctypes.c_float(scale), ctypes.c_int(win), _ptr(out), self._stream())
                self._done(rc, "paged_attention_prefill")
                kernel = "attention_prefill_cp_async"
            if trace.active():
                trace.note(kernel, *self._attention_work(batch, 0, batch.num_prefill_requests, nq,
                                                         nkv, hd, qkv.element_size(), win))
        tiles = batch.tiles[self.generic_q_tile]
        n_generic_tiles = 0 if tensor_core_prefill else tiles.shape[0]
        n_generic_decode = 0 if split else n_decode
        if n_generic_tiles + n_generic_decode > 0:
            rc = self.lib.somi_paged_attention_generic(
                _ptr(qkv), _code(qkv), ctypes.c_int(qkv.shape[1]), _ptr(kcache), _ptr(vcache),
                _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(n_generic_tiles),
                ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(batch.num_prefill_tokens),
                ctypes.c_int(n_generic_decode), ctypes.c_int(nq), ctypes.c_int(nkv),
                ctypes.c_int(hd), ctypes.c_int(vd), ctypes.c_int(page_size), ctypes.c_float(scale),
                ctypes.c_int(max(win, 0)), ctypes.c_int(chunk), _ptr(gate),
                ctypes.c_longlong(gate.stride(0) if gate is not None else 0),
                ctypes.c_int(1 if gate_per_head else 0), ctypes.c_float(cap), _ptr(sinks),
                _ptr(out), self._stream())
            self._done(rc, "paged_attention")
            if trace.active():
                first = batch.num_prefill_requests if tensor_core_prefill else 0
                last = batch.num_prefill_requests if split else batch.num_requests
                trace.note("attention_generic", *self._attention_work(
                    batch, first, last, nq, nkv, hd, qkv.element_size(), win))
        if split:
            chunk = self.decode_chunk
            max_splits = -(-group.width * page_size // chunk)
            n_o = n_decode * nq * max_splits * hd
            ws = self._scratch(n_o + n_decode * nq * max_splits * 2, qkv.device)
            tma = (not shaped and self.use_tma_decode and storage is not None and bool(
                self.lib.somi_decode_tma_supported(ctypes.c_int(nq), ctypes.c_int(nkv),
                                                   ctypes.c_int(hd), ctypes.c_int(page_size))))
            if tma:
                row_bytes = hd * 2
                k_row0 = (kcache.data_ptr() - storage.data_ptr()) // row_bytes
                v_row0 = (vcache.data_ptr() - storage.data_ptr()) // row_bytes
                rc = self.lib.somi_paged_attention_decode_tma(
                    ctypes.c_void_p(self._kv_tensor_map(storage, hd, page_size)), _ptr(qkv),
                    ctypes.c_int(qkv.shape[1]), ctypes.c_int(batch.num_prefill_tokens),
                    ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(n_decode),
                    ctypes.c_longlong(k_row0), ctypes.c_longlong(v_row0),
                    _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.ctx_len),
                    ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd),
                    ctypes.c_int(page_size), ctypes.c_float(scale), ctypes.c_int(win),
                    ctypes.c_void_p(ws.data_ptr()), ctypes.c_void_p(ws.data_ptr() + 4 * n_o),
                    ctypes.c_int(max_splits), _ptr(out), self._stream())
            else:
                rc = self.lib.somi_paged_attention_decode_shaped(
                    _ptr(qkv), ctypes.c_int(qkv.shape[1]), ctypes.c_int(batch.num_prefill_tokens),
                    ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(n_decode),
                    _ptr(kcache), _ptr(vcache), _ptr(group.block_table),
                    ctypes.c_int(group.width), _ptr(batch.ctx_len), ctypes.c_int(nq),
                    ctypes.c_int(nkv), ctypes.c_int(hd), ctypes.c_int(page_size),
                    ctypes.c_float(scale), ctypes.c_int(win), ctypes.c_float(cap), _ptr(sinks),
                    ctypes.c_void_p(ws.data_ptr()),
                    ctypes.c_void_p(ws.data_ptr() + 4 * n_o), ctypes.c_int(max_splits),
                    _ptr(out), self._stream())
            self._done(rc, "paged_attention_decode")
            if max_splits > 1:
                self.launches += 1
            if trace.active():
                trace.note("attention_decode_tma" if tma else "attention_decode_cp_async",
                           *self._attention_work(batch, batch.num_prefill_requests,
                                                 batch.num_requests, nq, nkv, hd,
                                                 qkv.element_size(), win),
                           detail="with merge" if max_splits > 1 else "")

        if gate is not None and (tensor_core_prefill or split):
            # the generic kernel applied the gate to its own rows only
            first = 0 if tensor_core_prefill else batch.num_prefill_tokens
            last = batch.num_tokens if split else batch.num_prefill_tokens
            if gate_per_head:
                rc = self.lib.somi_head_gate_mul(
                    _ptr(out[first:last]), _ptr(gate[first:last]), _code(out),
                    ctypes.c_longlong(gate.stride(0)), ctypes.c_longlong(last - first),
                    ctypes.c_int(nq), ctypes.c_int(vd), self._stream())
                self._done(rc, "head_gate_mul")
                if trace.active():
                    trace.note("head_gate_mul", 2 * (last - first) * nq * vd * out.element_size())
            else:
                self.sigmoid_gate_mul(out[first:last], gate[first:last])

    # ------------------------------------------------ gated layers, latent attention
    def embed_sinusoid_layernorm(self, ids, positions, table, inv_freq, weight, eps, out) -> None:
        """out = layernorm(table[ids] + sinusoid(positions)) * weight, float32 [T, H]."""
        _check(ids, positions, table, inv_freq, weight, out)
        assert ids.dtype == torch.int32 and positions.dtype == torch.int32
        assert out.dtype == torch.float32 and inv_freq.dtype == torch.float32
        assert inv_freq.numel() == (table.shape[1] + 1) // 2
        rc = self.lib.somi_embed_sinusoid_layernorm(
            _ptr(ids), _ptr(positions), _ptr(table), _code(table), _ptr(inv_freq), _ptr(weight),
            _code(weight), ctypes.c_float(eps), _ptr(out), ctypes.c_int(ids.shape[0]),
            ctypes.c_int(table.shape[1]), self._stream())
        self._done(rc, "embed_sinusoid_layernorm")
        if trace.active():
            trace.note("embed_sinusoid_layernorm", ids.shape[0] * table.shape[1] * (table.element_size() + 4))

    def add_layernorm(self, residual, delta, gate, weight, eps, out, rows=None, rms=False,
                      extra=None) -> None:
        """residual += sigmoid(gate) * delta (float32, in place; no gate: plain sum);
        out = layernorm(residual) * weight (mean taken off; with `rms`, an RMS norm instead).

        `delta`: [N, H] in the compute dtype, or float32 [splits, N, H] partial sums added in
        order.  `gate`: logits [N, H] whose rows may lie further apart (a view of a wider
        product), or float32 [splits, N, H] partial sums.  `extra`: float32 [N, H] rows that are
        added as well, outside the gate (a second branch of the layer; needs a `delta`).  With
        `rows`, only those rows are produced and residual is not written."""
        _check(residual, delta, weight, out, rows, extra)
        assert residual.dtype == torch.float32
        assert extra is None or (extra.dtype == torch.float32 and extra.shape == residual.shape
                                 and delta is not None)
        H = residual.shape[1]
        n_out = out.shape[0]
        splits, stride = 1, 0
        if delta is not None and delta.dim() == 3:
            assert delta.dtype == torch.float32
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        gate_stride, gate_splits, gate_split_stride = 0, 1, 0
        if gate is not None:
            if gate.dim() == 3:          # float32 partial sums of a split-K product
                if not (gate.is_cuda and gate.is_contiguous() and gate.dtype == torch.float32
                        and tuple(gate.shape[1:]) == (residual.shape[0], H)):
                    raise KernelError("partial sums of a gate are contiguous float32 [splits, rows, H]")
                gate_splits, gate_split_stride, gate_stride = gate.shape[0], gate.shape[1] * H, H
            else:
                if not gate.is_cuda or gate.stride(1) != 1 or gate.shape != (residual.shape[0], H):
                    raise KernelError("a gate is [rows, H] with contiguous rows")
                gate_stride = gate.stride(0)
        rc = self.lib.somi_add_layernorm(
            _ptr(residual), _ptr(delta), _code(delta) if delta is not None else _code(out),
            ctypes.c_int(splits), ctypes.c_longlong(stride), _ptr(gate),
            _code(gate) if gate is not None else _code(out), ctypes.c_longlong(gate_stride),
            ctypes.c_int(gate_splits), ctypes.c_longlong(gate_split_stride),
            _ptr(weight), _code(weight), ctypes.c_float(eps), _ptr(out), _code(out), _ptr(rows),
            ctypes.c_int(n_out), ctypes.c_int(H), ctypes.c_int(0 if rows is not None else 1),
            ctypes.c_int(1 if rms else 0), _ptr(extra), self._stream())
        self._done(rc, "add_layernorm")
        if trace.active():
            n = n_out * H
            moved = n * (4 + out.element_size()) + H * weight.element_size()
            if delta is not None:
                moved += splits * n * delta.element_size()
            if gate is not None:
                moved += gate_splits * n * gate.element_size()
            if extra is not None:
                moved += n * 4
            if rows is None:
                moved += n * 4
            trace.note("add_layernorm", moved, detail=f"splits={splits}" if splits > 1 else "")

    def check_taps(self, taps: int) -> None:
        if not 1 <= taps <= self.max_taps:
            raise KernelError(f"a causal convolution of {taps} taps is not supported (1 to "
                              f"{self.max_taps})")

    def causal_taps(self, h, weight, state, batch, out) -> None:
        """out = h + conv(h) over each request's rows (`weight`: float32 [taps, H], the newest
        input's tap last), continued from `state` [slots, taps-1, H] (the request's last inputs),
        which is moved on by this step's rows."""
        _check(h, weight, state, out)
        taps = weight.shape[0]
        assert weight.dtype == torch.float32 and weight.shape[1] == h.shape[1]
        if taps > 1:
            assert state is not None and state.dtype == h.dtype
            assert tuple(state.shape[1:]) == (taps - 1, h.shape[1])
        rc = self.lib.somi_causal_taps(
            _ptr(h), _code(h), _ptr(weight), _ptr(state), _ptr(batch.cu_q),
            _ptr(batch.token_request), _ptr(batch.state_slot), _ptr(out), ctypes.c_int(h.shape[0]),
            ctypes.c_int(batch.num_requests), ctypes.c_int(h.shape[1]), ctypes.c_int(taps),
            self._stream())
        self._done(rc, "causal_taps")
        if taps > 1 and not (h.shape[0] == batch.num_requests and h.shape[1] % 4 == 0):
            self.launches += 1      # the state's own kernel (a step of single tokens needs none)
        if trace.active():
            trace.note("causal_taps", 2 * h.numel() * h.element_size()
                       + 2 * batch.num_requests * (taps - 1) * h.shape[1] * h.element_size())

    def latent_norm_store(self, x, na, nb, wa, wb, eps, a_out, slot_map, cache) -> None:
        """x = [a | b] per row: a_out = rmsnorm(a) * wa; rmsnorm(b) * wb goes to the cache slot of
        the row's token (`nb` = 0: there is no b).  x: [T, na + nb], or float32 [splits, T, na + nb]
        partial sums that are added up in order."""
        _check(x, wa, wb, a_out, slot_map, cache)
        splits, split_stride = 1, 0
        if x.dim() == 3:                 # float32 partial sums of a split-K product
            assert x.dtype == torch.float32
            splits, split_stride = x.shape[0], x.shape[1] * x.shape[2]
        assert x.shape[-1] == na + nb and (a_out.dtype == x.dtype or x.dtype == torch.float32)
        if nb:
            assert cache.dtype == a_out.dtype and cache.shape[-1] == nb and cache.shape[1] == 1
            assert wb.dtype == wa.dtype
        rc = self.lib.somi_latent_norm_store(
            _ptr(x), _code(x), ctypes.c_longlong(x.shape[-1]), ctypes.c_int(splits),
            ctypes.c_longlong(split_stride), ctypes.c_int(na), ctypes.c_int(nb),
            _ptr(wa), _ptr(wb), _code(wa), ctypes.c_float(eps), _ptr(a_out), _code(a_out),
            _ptr(slot_map), _ptr(cache), ctypes.c_int(a_out.shape[0]), self._stream())
        self._done(rc, "latent_norm_store")
        if trace.active():
            trace.note("latent_norm_store", x.numel() * x.element_size()
                       + a_out.shape[0] * (na + nb) * a_out.element_size(),
                       detail=f"splits={splits}" if splits > 1 else "")

    def xielu(self, x, n, act, out) -> None:
        """out[:, :n] = xielu(x[:, :n]) with (p, q) = act; x's rows may be wider than n."""
        _check(x, act, out)
        assert out.shape == (x.shape[0], n) and out.dtype == x.dtype and x.shape[1] >= n
        rc = self.lib.somi_xielu(_ptr(x), _code(x), ctypes.c_longlong(x.shape[1]), _ptr(act),
                                 _code(act), _ptr(out), ctypes.c_int(x.shape[0]), ctypes.c_int(n),
                                 self._stream())
        self._done(rc, "xielu")
        if trace.active():
            trace.note("xielu", 2 * out.numel() * out.element_size())

    def head_product(self, x: torch.Tensor, w: torch.Tensor, heads_first: bool) -> torch.Tensor:
        """A product per head: y_h = x_h @ w_h^T with w [heads, N, K].

        `heads_first`: x is [T, heads, K] (a view of a [T, heads * K] projection) and y comes
        back as [heads, T, N]; otherwise x is [heads, T, K] and y is [T, heads, N], so that the
        next projection reads [T, heads * N] without a copy.  float32: the engine's own product,
        batched over heads; bfloat16: the library's batched product."""
        H, N, K = w.shape
        if heads_first:
            T = x.shape[0]
            xs = x.transpose(0, 1)                               # [H, T, K] view
            y = torch.empty((H, T, N), dtype=x.dtype, device=x.device)
            ys = y
        else:
            T = x.shape[1]
            xs = x
            y = torch.empty((T, H, N), dtype=x.dtype, device=x.device)
            ys = y.transpose(0, 1)                               # [H, T, N] view
        assert xs.shape == (H, T, K) and xs.stride(2) == 1 and w.is_contiguous()
        if x.dtype == torch.float32:
            rc = self.lib.somi_gemm_f32_batched(
                _ptr(xs), _ptr(w), None, _ptr(ys), ctypes.c_int(T), ctypes.c_int(N),
                ctypes.c_int(K), ctypes.c_int(H), ctypes.c_longlong(xs.stride(1)),
                ctypes.c_longlong(ys.stride(1)), ctypes.c_longlong(xs.stride(0)),
                ctypes.c_longlong(N * K), ctypes.c_longlong(ys.stride(0)), self._stream())
            self._done(rc, "gemm_f32_batched")
            name = "gemm_f32_batched"
        else:
            torch.bmm(xs, w.transpose(1, 2), out=ys)
            name = "library_gemm_batched"
        if trace.active():
            trace.note(name, (H * N * K + 2 * T * H * K) * x.element_size(), 2.0 * T * H * N * K,
                       detail=f"heads={H} M={T} N={N} K={K}")
        return y

    def check_latent_geometry(self, heads: int, rank: int) -> None:
        if not (1 <= rank <= 512 and 1 <= heads <= 65535):
            raise KernelError(f"latent attention over a latent of {rank} elements with {heads} "
                              "heads is not supported (latent up to 512)")

    def latent_attention(self, q, cache, batch, group, heads, rank, scale, window, sinks, out) -> None:
        """Attention of every token of the step over a cache of latents that serve as keys and
        as values for every head (`q`, `out`: [heads, T, rank]; cache [pages, 1, page, rank]);
        `sinks`: float32 [heads] scores that join every softmax's denominator, or None."""
        _check(q, cache, out, group.block_table, sinks)
        assert q.dtype == cache.dtype == out.dtype and q.shape == out.shape == (heads, q.shape[1], rank)
        assert cache.shape[1] == 1 and cache.shape[3] == rank
        assert sinks is None or (sinks.dtype == torch.float32 and sinks.numel() == heads)
        page_size = cache.shape[2]
        T = q.shape[1]
        tiles = batch.tiles[self.latent_q_tile]
        n_decode = batch.num_requests - batch.num_prefill_requests
        win = int(window) if window else 0
        if (self.use_mma_latent and q.dtype == torch.bfloat16
                and bool(self.lib.somi_latent_attention_mma_supported(ctypes.c_int(heads),
                                                                      ctypes.c_int(rank)))):
            # tensor cores: 16 tokens x 4 heads per CTA for prompt portions; all heads of a
            # single-token request per CTA, its keys in chunks whose partial sums are merged
            max_kv = group.width * page_size      # a bound that changes with the layout only
            splits = int(self.lib.somi_latent_attention_mma_splits(
                ctypes.c_int(max_kv), ctypes.c_int(win), ctypes.c_int(n_decode), ctypes.c_int(heads)))
            ws = self._scratch(n_decode * heads * splits * (rank + 2), q.device) if splits > 1 and n_decode else None
            rc = self.lib.somi_latent_attention_mma(
                _ptr(q), ctypes.c_longlong(rank), ctypes.c_longlong(T * rank), _ptr(cache),
                _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
                _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]),
                ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(batch.num_prefill_tokens),
                ctypes.c_int(n_decode), ctypes.c_int(max_kv), ctypes.c_int(heads),
                ctypes.c_int(rank), ctypes.c_int(page_size), ctypes.c_float(scale),
                ctypes.c_int(win), _ptr(sinks), _ptr(out), ctypes.c_longlong(rank),
                ctypes.c_longlong(T * rank), _ptr(ws), self._stream())
            self._done(rc, "latent_attention_mma")
            self.launches += (1 if tiles.shape[0] and n_decode else 0) + (1 if splits > 1 and n_decode else 0)
            if trace.active():
                moved, flops = self._attention_work(batch, 0, batch.num_requests, heads, 1, rank,
                                                    q.element_size(), win)
                trace.note("latent_attention_mma", moved / 2 + heads * T * rank * q.element_size(), flops,
                           detail=f"splits={splits}" if n_decode else "")
            return
        rc = self.lib.somi_latent_attention_generic(
            _ptr(q), _code(q), ctypes.c_longlong(rank), ctypes.c_longlong(T * rank), _ptr(cache),
            _ptr(group.block_table), ctypes.c_int(group.width), _ptr(batch.cu_q),
            _ptr(batch.ctx_len), _ptr(tiles), ctypes.c_int(tiles.shape[0]),
            ctypes.c_int(batch.num_prefill_requests), ctypes.c_int(batch.num_prefill_tokens),
            ctypes.c_int(n_decode), ctypes.c_int(heads), ctypes.c_int(rank),
            ctypes.c_int(page_size), ctypes.c_float(scale), ctypes.c_int(int(window) if window else 0),
            _ptr(sinks), _ptr(out), ctypes.c_longlong(rank), ctypes.c_longlong(T * rank),
            self._stream())
        self._done(rc, "latent_attention")
        if trace.active():
            moved, flops = self._attention_work(batch, 0, batch.num_requests, heads, 1, rank,
                                                q.element_size(), int(window) if window else 0)
            trace.note("latent_attention_generic", moved / 2 + heads * T * rank * q.element_size(), flops)

    # ------------------------------- sandwich norms, convolutions, pair rotation, recurrence
    def embed_scaled(self, ids, table, scale: float, out) -> None:
        """out = float32(table[ids]) * scale."""
        _check(ids, table, out)
        assert ids.dtype == torch.int32 and out.dtype == torch.float32
        rc = self.lib.somi_embed_scaled(_ptr(ids), _ptr(table), _code(table), ctypes.c_float(scale),
                                        _ptr(out), ctypes.c_int(ids.shape[0]),
                                        ctypes.c_int(table.shape[1]), self._stream())
        self._done(rc, "embed_scaled")
        if trace.active():
            trace.note("embed", ids.shape[0] * table.shape[1] * (table.element_size() + 4))

    def add_normed_rmsnorm(self, residual, delta, weight_b, eps_b, weight, eps, out, rows=None) -> None:
        """residual += rmsnorm(delta) * weight_b (float32, in place), then, where `out` is given,
        out = rmsnorm(residual) * weight.  `delta`: [N, H], or float32 [splits, N, H] partial sums
        added in order, or None (nothing is added).  With `rows`, only those rows are produced and
        residual is not written."""
        _check(residual, delta, weight_b, weight, out, rows)
        assert residual.dtype == torch.float32
        H = residual.shape[1]
        n_out = residual.shape[0] if rows is None else rows.shape[0]
        splits, stride = 1, 0
        if delta is not None and delta.dim() == 3:
            assert delta.dtype == torch.float32
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        rc = self.lib.somi_add_normed_rmsnorm(
            _ptr(residual), _ptr(delta), _code(delta) if delta is not None else _F32,
            ctypes.c_int(splits), ctypes.c_longlong(stride), _ptr(weight_b),
            _code(weight_b) if weight_b is not None else _F32, ctypes.c_float(eps_b), _ptr(weight),
            _code(weight) if weight is not None else _F32, ctypes.c_float(eps), _ptr(out),
            _code(out) if out is not None else _F32, _ptr(rows), ctypes.c_int(n_out), ctypes.c_int(H),
            ctypes.c_int(0 if rows is not None else 1), self._stream())
        self._done(rc, "add_normed_rmsnorm")
        if trace.active():
            n = n_out * H
            moved = n * 4
            if out is not None:
                moved += n * out.element_size()
            if delta is not None:
                moved += splits * n * delta.element_size() + (n * 4 if rows is None else 0)
            trace.note("add_normed_rmsnorm", moved, detail=f"splits={splits}" if splits > 1 else "")

    def check_conv_taps(self, taps: int) -> None:
        most = int(self.lib.somi_causal_conv_max_taps())
        if not 1 <= taps <= most:
            raise KernelError(f"a causal convolution of {taps} taps is not supported (1 to {most})")

    def causal_conv(self, u, channels, weight, bias, state, batch, out, act=None,
                    add_input=False) -> None:
        """out[:, :channels] = act(bias + conv(u[:, :channels])) (+ u) over each request's rows.
        `u` and `out` may be views whose rows are wider than `channels`; `weight`: float32
        [taps, channels], the newest input's tap last; `state` [slots, taps - 1, channels] holds
        each request's last inputs and is moved on by this step's rows.  act: None or "silu"."""
        _check(weight, bias, state)
        taps = weight.shape[0]
        if not (u.is_cuda and out.is_cuda and u.stride(1) == 1 and out.stride(1) == 1
                and u.dtype == out.dtype and u.shape[1] >= channels and out.shape[1] >= channels):
            raise KernelError("causal_conv takes device tensors with contiguous rows")
        assert weight.dtype == torch.float32 and weight.shape[1] == channels
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == channels)
        if taps > 1:
            assert state is not None and state.dtype == u.dtype
            assert tuple(state.shape[1:]) == (taps - 1, channels)
        rc = self.lib.somi_causal_conv(
            _ptr(u), _code(u), ctypes.c_longlong(u.stride(0)), _ptr(weight), _ptr(bias), _ptr(state),
            _ptr(batch.cu_q), _ptr(batch.token_request), _ptr(batch.state_slot), _ptr(out),
            ctypes.c_longlong(out.stride(0)), ctypes.c_int(u.shape[0]),
            ctypes.c_int(batch.num_requests), ctypes.c_int(channels), ctypes.c_int(taps),
            ctypes.c_int({None: 0, "silu": 1}[act]), ctypes.c_int(1 if add_input else 0),
            self._stream())
        self._done(rc, "causal_conv")
        if taps > 1:
            self.launches += 1
        if trace.active():
            trace.note("causal_conv", 2 * u.shape[0] * channels * u.element_size()
                       + 2 * batch.num_requests * (taps - 1) * channels * u.element_size())

    def rotary_pairs_store(self, qkv, positions, inv_freq, nq, nkv, hd, vd, rotary_dim, unit_norm,
                           eps, slot_map, kcache, vcache) -> None:
        """Rows of `qkv` hold nq query heads and nkv key heads of `hd` elements, then nkv value
        heads of `vd`.  Neighbouring pairs (2i, 2i+1) below `rotary_dim` of every query and key
        head turn by position * inv_freq[i] (`inv_freq` float64: the angle is reduced in float64, its
        sine and cosine are float32); with `unit_norm` each head is then divided by its
        root mean square (eps inside the root).  Queries are rewritten in place; keys and values
        go to their cache slots (`slot_map` None: nothing is stored)."""
        _check(positions, inv_freq, slot_map, kcache, vcache)
        if not (qkv.is_cuda and qkv.stride(1) == 1 and qkv.shape[1] >= (nq + nkv) * hd + nkv * vd):
            raise KernelError("rotary_pairs_store takes a device tensor with contiguous rows")
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() >= max(1, rotary_dim // 2)
        page_size = 1
        if slot_map is not None:
            assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
            assert kcache.shape[1] == nkv and kcache.shape[3] == hd and vcache.shape[3] == vd
            page_size = kcache.shape[2]
        rc = self.lib.somi_rotary_pairs_store(
            _ptr(qkv), _code(qkv), ctypes.c_longlong(qkv.stride(0)), _ptr(positions), _ptr(inv_freq),
            ctypes.c_int(qkv.shape[0]), ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd),
            ctypes.c_int(vd), ctypes.c_int(rotary_dim), ctypes.c_int(1 if unit_norm else 0),
            ctypes.c_float(eps), _ptr(slot_map), _ptr(kcache), _ptr(vcache),
            ctypes.c_int(page_size), self._stream())
        self._done(rc, "rotary_pairs_store")
        if trace.active():
            n = qkv.shape[0] * ((nq + nkv) * hd + nkv * vd)
            trace.note("rotary_pairs_store", 2 * n * qkv.element_size())

    def sigmoid_gate_mul(self, x, gate) -> None:
        """x *= sigmoid(gate) (float32 arithmetic); `gate`'s rows may lie further apart."""
        if not (x.is_cuda and x.is_contiguous() and gate.is_cuda and gate.stride(1) == 1
                and gate.shape == x.shape and gate.dtype == x.dtype):
            raise KernelError("sigmoid_gate_mul takes a contiguous x and a gate with contiguous rows")
        rc = self.lib.somi_sigmoid_gate_mul(_ptr(x), _ptr(gate), _code(x),
                                            ctypes.c_longlong(gate.stride(0)),
                                            ctypes.c_longlong(x.shape[0]), ctypes.c_int(x.shape[1]),
                                            self._stream())
        self._done(rc, "sigmoid_gate_mul")
        if trace.active():
            trace.note("sigmoid_gate_mul", 3 * x.numel() * x.element_size())

    def softcap(self, x, cap: float) -> None:
        """x = cap * tanh(x / cap), in place (float32)."""
        _check(x)
        assert x.dtype == torch.float32
        rc = self.lib.somi_softcap(_ptr(x), ctypes.c_float(cap), ctypes.c_longlong(x.numel()),
                                   self._stream())
        self._done(rc, "softcap")
        if trace.active():
            trace.note("softcap", 8 * x.numel())

    def check_ssm_geometry(self, heads: int, groups: int, state: int) -> None:
        most = int(self.lib.somi_ssm_scan_max_state())
        if not (1 <= state <= most and groups >= 1 and heads % groups == 0):
            raise KernelError(f"a state-space mixer with {heads} heads in {groups} groups and a "
                              f"state of {state} is not supported (state up to {most})")

    def ssm_scan(self, xbc, dt_raw, dt_bias, a_log, skip, state, batch, y, heads, groups, n_state,
                 vdim) -> None:
        """The recurrence of a state-space mixer over each request's rows, continued from and
        left in `state` (float32 [slots, heads, vdim, n_state]); `xbc` rows hold x, B, C; `dt_raw`
        [T, heads] (a view of wider rows); y: float32 [T, heads * vdim]."""
        _check(dt_bias, a_log, skip, state, y)
        if not (xbc.is_cuda and xbc.stride(1) == 1 and dt_raw.is_cuda and dt_raw.stride(1) == 1
                and dt_raw.dtype == xbc.dtype):
            raise KernelError("ssm_scan takes device tensors with contiguous rows")
        assert state.dtype == y.dtype == dt_bias.dtype == a_log.dtype == skip.dtype == torch.float32
        assert tuple(state.shape[1:]) == (heads, vdim, n_state)
        assert xbc.shape[1] >= heads * vdim + 2 * groups * n_state
        rc = self.lib.somi_ssm_scan(
            _ptr(xbc), _code(xbc), ctypes.c_longlong(xbc.stride(0)), _ptr(dt_raw),
            ctypes.c_longlong(dt_raw.stride(0)), _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(state),
            _ptr(batch.cu_q), _ptr(batch.state_slot), _ptr(y), ctypes.c_int(batch.num_requests),
            ctypes.c_int(heads), ctypes.c_int(groups), ctypes.c_int(n_state), ctypes.c_int(vdim),
            self._stream())
        self._done(rc, "ssm_scan")
        if trace.active():
            T = xbc.shape[0]
            trace.note("ssm_scan", T * (heads * vdim + 2 * groups * n_state) * xbc.element_size()
                       + T * heads * vdim * 4 + 2 * batch.num_requests * heads * n_state * vdim * 4,
                       6.0 * T * heads * n_state * vdim)

    def gated_group_rmsnorm(self, y, z, weight, eps, groups, out) -> None:
        """out = rmsnorm over each of `groups` equal parts of y * silu(z), times weight."""
        _check(y, weight, out)
        if not (z.is_cuda and z.stride(1) == 1 and z.shape == y.shape and z.dtype == out.dtype):
            raise KernelError("gated_group_rmsnorm takes a gate with contiguous rows")
        assert y.dtype == torch.float32
        rc = self.lib.somi_gated_group_rmsnorm(
            _ptr(y), _ptr(z), _code(z), ctypes.c_longlong(z.stride(0)), _ptr(weight), _code(weight),
            ctypes.c_float(eps), _ptr(out), ctypes.c_int(y.shape[0]), ctypes.c_int(y.shape[1]),
            ctypes.c_int(groups), self._stream())
        self._done(rc, "gated_group_rmsnorm")
        if trace.active():
            trace.note("gated_group_rmsnorm", y.numel() * (4 + 2 * out.element_size()))

    # ------------------------------------------------------------ mixture of experts
    def moe_route(self, token_ids, table, num_experts: int, all_experts: int | None = None
                  ) -> tuple[torch.Tensor, int]:
        """Group the step's (token, k) entries by the expert that `table` [vocab, top] gives each
        token id (`token_ids` None: `table` [T, top] holds the step's own rows, as a router wrote
        them).  Experts numbered `num_experts` up to `all_experts` have no matrices: their entries
        are placed behind the others and get no tile.  Returns the device work area that
        `grouped_product` reads and its tile bound."""
        _check(token_ids, table)
        assert (token_ids is None or token_ids.dtype == torch.int32) and table.dtype == torch.int32
        T = table.shape[0] if token_ids is None else token_ids.shape[0]
        top = table.shape[1]
        bm = int(self.lib.somi_moe_row_tile())
        max_tiles = -(-T * top // bm) + num_experts
        work = torch.empty(num_experts + 1 + 2 * T * top + 2 * max_tiles + 1, dtype=torch.int32,
                           device=table.device)
        rc = self.lib.somi_moe_route(_ptr(token_ids), _ptr(table), ctypes.c_int(T), ctypes.c_int(top),
                                     ctypes.c_int(num_experts),
                                     ctypes.c_int(all_experts if all_experts else num_experts),
                                     _ptr(work), ctypes.c_int(max_tiles), self._stream())
        self._done(rc, "moe_route")
        if trace.active():
            trace.note("moe_route", 12 * T * top)
        return work, max_tiles

    ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "silu": 2, "relu2": 3}

    def grouped_product(self, a, w, *, route=None, top=1, gather=False, scatter=False,
                        gated=None, out_float32=False, act=None) -> torch.Tensor:
        """Rows of `a` times the matrix of their group: w [E, N, K].

        `route` = (work, max_tiles) from `moe_route` (None: one group, w [1, N, K], all rows).
        `gather`: row p of the grouped order reads a[entry(p) // top] (else a[p]); `scatter`: it
        writes out[entry(p)] (else out[p]).  `gated` = (limit, alpha[, shift = 1]): w's rows
        alternate gate, up and the result is g * sigmoid(alpha * g) * (u + shift) with
        g = min(gate, limit), u = clamp(up, -limit, limit), N / 2 columns wide (limit infinite,
        alpha 1, shift 0: silu(gate) * up).  `act` (a name of `ACTIVATIONS`): the result is that
        function of the product, N columns wide (an expert without a gate).  Products are float32
        FMAs summed over K in ascending order."""
        _check(a, w)
        E, N, K = w.shape
        assert a.shape[1] == K and a.dtype == w.dtype
        if route is None:
            assert E == 1
            work, max_tiles, n_entries, n_rows = None, 0, 0, a.shape[0]
        else:
            work, max_tiles = route
            n_entries = (work.numel() - (E + 1) - 2 * max_tiles - 1) // 2
            n_rows = n_entries
        cols = N // 2 if gated is not None else N
        assert gated is None or act is None
        out_dtype = torch.float32 if (out_float32 and gated is None and act is None) else a.dtype
        out = torch.empty((n_rows, cols), dtype=out_dtype, device=a.device)
        limit, alpha, shift = self._gated(gated)
        mode = 1 if gated is not None else (2 if act is not None else 0)
        rc = self.lib.somi_grouped_gemm(
            _ptr(a), _code(a), ctypes.c_longlong(a.stride(0)), ctypes.c_int(top),
            ctypes.c_int(1 if gather else 0), _ptr(w), _ptr(work), ctypes.c_int(E),
            ctypes.c_int(n_entries), ctypes.c_int(max_tiles), ctypes.c_int(n_rows), _ptr(out),
            ctypes.c_int(1 if out_dtype == torch.float32 else 0), ctypes.c_longlong(cols),
            ctypes.c_int(1 if scatter else 0), ctypes.c_int(N), ctypes.c_int(K),
            ctypes.c_int(mode), ctypes.c_float(limit), ctypes.c_float(alpha),
            ctypes.c_float(shift), ctypes.c_int(self.ACTIVATIONS[act] if act is not None else 0),
            self._stream())
        self._done(rc, "grouped_product")
        if trace.active():
            trace.note("grouped_product", (min(E, n_rows) * N * K + n_rows * K) * a.element_size()
                       + out.numel() * out.element_size(), 2.0 * n_rows * N * K,
                       detail=f"E={E} rows={n_rows} N={N} K={K}")
        return out

    @staticmethod
    def _gated(gated) -> tuple[float, float, float]:
        """(limit, alpha, shift) of a gated activation; the shift is 1 where it is not given."""
        if gated is None:
            return 0.0, 0.0, 0.0
        return float(gated[0]), float(gated[1]), float(gated[2]) if len(gated) > 2 else 1.0

    @staticmethod
    def _route_parts(route, E: int):
        """(offsets [E + 1], sorted [n], place [n]) views of a work area of `moe_route`."""
        work, max_tiles = route
        n = (work.numel() - (E + 1) - 2 * max_tiles - 1) // 2
        return work[:E + 1], work[E + 1:E + 1 + n], work[work.numel() - n:]

    def moe_gather_rows(self, a, route, E: int, top: int) -> torch.Tensor:
        """The step's rows in the grouped order: out[p] = a[entry(p) // top]."""
        _check(a)
        work, _ = route
        n = self._route_parts(route, E)[1].numel()
        out = torch.empty((n, a.shape[1]), dtype=a.dtype, device=a.device)
        rc = self.lib.somi_moe_gather_rows(_ptr(a), _code(a), ctypes.c_longlong(a.stride(0)), _ptr(work),
                                           ctypes.c_int(E), ctypes.c_int(n), ctypes.c_int(top),
                                           ctypes.c_int(a.shape[1]), _ptr(out), self._stream())
        self._done(rc, "moe_gather_rows")
        if trace.active():
            trace.note("moe_gather_rows", 2 * out.numel() * out.element_size())
        return out

    def clamped_gate_up(self, gu, limit: float, alpha: float, shift: float = 1.0) -> torch.Tensor:
        """Columns of `gu` alternate gate, up: g * sigmoid(alpha * g) * (u + shift) with
        g = min(gate, limit), u = clamp(up, -limit, limit); float32 arithmetic."""
        _check(gu)
        ff = gu.shape[1] // 2
        out = torch.empty((gu.shape[0], ff), dtype=gu.dtype, device=gu.device)
        rc = self.lib.somi_clamped_gate_up(_ptr(gu), _ptr(out), _code(gu), ctypes.c_longlong(gu.shape[0]),
                                           ctypes.c_int(ff), ctypes.c_float(limit), ctypes.c_float(alpha),
                                           ctypes.c_float(shift), self._stream())
        self._done(rc, "clamped_gate_up")
        if trace.active():
            trace.note("clamped_gate_up", 3 * out.numel() * out.element_size())
        return out

    def unary_act(self, x, act: str) -> torch.Tensor:
        """`act` (a name of `ACTIVATIONS`) of every element, float32 arithmetic."""
        _check(x)
        out = torch.empty_like(x)
        rc = self.lib.somi_unary_act(_ptr(x), _ptr(out), _code(x), ctypes.c_longlong(x.numel()),
                                     ctypes.c_int(self.ACTIVATIONS[act]), self._stream())
        self._done(rc, "unary_act")
        if trace.active():
            trace.note("unary_act", 2 * x.numel() * x.element_size())
        return out

    def add_concat(self, residual, delta, extra, tail, out) -> None:
        """out = [residual + delta + extra | tail] in out's dtype, [N, 2 H]; residual, tail and
        extra float32 [N, H]; `delta`: [N, H], or float32 [splits, N, H] partial sums added in
        order, or None (then there is no extra either).  Nothing but `out` is written."""
        _check(residual, delta, extra, tail, out)
        assert residual.dtype == tail.dtype == torch.float32 and residual.shape == tail.shape
        assert extra is None or (extra.dtype == torch.float32 and delta is not None)
        N, H = residual.shape
        assert tuple(out.shape) == (N, 2 * H)
        splits, stride = 1, 0
        if delta is not None and delta.dim() == 3:
            assert delta.dtype == torch.float32
            splits, stride = delta.shape[0], delta.shape[1] * delta.shape[2]
        rc = self.lib.somi_add_concat(
            _ptr(residual), _ptr(delta), _code(delta) if delta is not None else _code(out),
            ctypes.c_int(splits), ctypes.c_longlong(stride), _ptr(extra), _ptr(tail), _ptr(out),
            _code(out), ctypes.c_int(N), ctypes.c_int(H), self._stream())
        self._done(rc, "add_concat")
        if trace.active():
            moved = N * H * (8 + 2 * out.element_size())
            if delta is not None:
                moved += splits * N * H * delta.element_size()
            if extra is not None:
                moved += N * H * 4
            trace.note("add_concat", moved)

    def moe_gemv_supported(self, n_entries: int, K: int, dtype) -> bool:
        """Whether a step's entries are few enough (and the sizes fit) for each to stream its
        expert's rows by itself."""
        return dtype == torch.bfloat16 and n_entries <= 64 and K % 8 == 0 and K <= 40 * 1024

    def moe_gemv(self, a, w, token_ids, table, *, per_token: bool, gated=None, act=None) -> torch.Tensor:
        """A step of few tokens: entry e = (token, k) times the matrix of expert
        table[id[token], k]; w [E, N, K] bfloat16.  `per_token`: a has one row per token (else one
        per entry).  `gated` = (limit, alpha): rows of w alternate gate, up and the result is the
        experts' activation, bfloat16 [entries, N / 2]; `act` (a name of `ACTIVATIONS`): that
        function of the product, bfloat16 [entries, N]; else float32 [entries, N]."""
        _check(a, w, token_ids, table)
        E, N, K = w.shape
        top = table.shape[1]
        n_tokens = table.shape[0] if token_ids is None else token_ids.shape[0]
        n = n_tokens * top
        assert a.dtype == w.dtype == torch.bfloat16 and a.shape[1] == K
        assert a.shape[0] == (n_tokens if per_token else n)
        assert gated is None or act is None
        if gated is not None:
            out = torch.empty((n, N // 2), dtype=torch.bfloat16, device=a.device)
        elif act is not None:
            out = torch.empty((n, N), dtype=torch.bfloat16, device=a.device)
        else:
            out = torch.empty((n, N), dtype=torch.float32, device=a.device)
        limit, alpha, shift = self._gated(gated)
        mode = 1 if gated is not None else (2 if act is not None else 0)
        rc = self.lib.somi_moe_gemv(
            _ptr(a), ctypes.c_longlong(a.stride(0)), ctypes.c_int(top if per_token else 1), _ptr(w),
            _ptr(token_ids), _ptr(table), ctypes.c_int(top), ctypes.c_int(E), ctypes.c_int(n),
            _ptr(out), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(mode),
            ctypes.c_float(limit), ctypes.c_float(alpha), ctypes.c_float(shift),
            ctypes.c_int(self.ACTIVATIONS[act] if act is not None else 0), self._stream())
        self._done(rc, "moe_gemv")
        if trace.active():
            trace.note("moe_gemv", (min(E, n) * N * K + n * K) * 2 + out.numel() * out.element_size(),
                       2.0 * n * N * K, detail=f"E={E} entries={n} N={N} K={K}")
        return out

    def library_grouped_product(self, a_sorted, w, route) -> torch.Tensor | None:
        """a_sorted [n, K] (rows in the grouped order) times w [E, N, K] by group, through the
        library's grouped product (bfloat16, prompt-sized steps); None where this build of the
        library has none for these sizes (asked once per shape class)."""
        E, N, K = w.shape
        if a_sorted.dtype != torch.bfloat16 or K % 8 or N % 8 or not hasattr(torch, "_grouped_mm"):
            return None
        if getattr(self, "_grouped_mm_broken", False):
            return None
        offsets = self._route_parts(route, E)[0][1:]
        try:
            out = torch._grouped_mm(a_sorted, w.transpose(1, 2), offs=offsets)
        except (RuntimeError, TypeError, NotImplementedError):
            if torch.cuda.is_current_stream_capturing():
                raise
            self._grouped_mm_broken = True
            return None
        if trace.active():
            n = a_sorted.shape[0]
            trace.note("library_grouped_gemm", (min(E, n) * N * K + n * K + n * N) * 2, 2.0 * n * N * K,
                       detail=f"E={E} rows={n} N={N} K={K}")
        return out

    def moe_combine(self, y, extra, weight: float, top: int, place=None) -> torch.Tensor:
        """out[t] = weight * sum_k y[row(t * top + k)] (+ extra[t]); float32.  `place`: int32, the
        row of every entry where y's rows are in the grouped order (else row = entry)."""
        _check(y, extra, place)
        assert extra is None or extra.dtype == torch.float32
        T, H = y.shape[0] // top, y.shape[1]
        out = torch.empty((T, H), dtype=torch.float32, device=y.device)
        rc = self.lib.somi_moe_combine(_ptr(y), _code(y), _ptr(place), _ptr(extra), ctypes.c_float(weight),
                                       ctypes.c_int(top), ctypes.c_int(T), ctypes.c_int(H), _ptr(out),
                                       self._stream())
        self._done(rc, "moe_combine")
        if trace.active():
            trace.note("moe_combine", y.numel() * y.element_size()
                       + (out.numel() + (0 if extra is None else extra.numel())) * 4)
        return out

    # ------------------------------- side-by-side branches, matrix-state mixers, routers
    def add_scaled_rmsnorm(self, residual, a, scale_a, b, scale_b, mult: float, extra, w1, w2,
                           eps: float, out1, out2, rows=None) -> None:
        """residual += mult * (scale_a * a + scale_b * b) + extra (float32, in place); then
        out1 = rmsnorm(residual) * w1 and out2 = rmsnorm(residual) * w2 (each where given).
        `a`, `b`: [N, H], or float32 [splits, N, H] partial sums added in order, or None; the
        scales are [H] or None; `extra` float32 [N, H] or None.  With `rows`, only those rows are
        produced and the residual is not written."""
        _check(residual, a, scale_a, b, scale_b, extra, w1, w2, out1, out2, rows)
        assert residual.dtype == torch.float32 and (extra is None or extra.dtype == torch.float32)
        H = residual.shape[1]
        n_out = residual.shape[0] if rows is None else rows.shape[0]

        def parts(d):
            if d is None:
                return _F32, 1, 0
            if d.dim() == 3:
                assert d.dtype == torch.float32
                return _F32, d.shape[0], d.shape[1] * d.shape[2]
            return _code(d), 1, 0

        (a_code, a_splits, a_stride), (b_code, b_splits, b_stride) = parts(a), parts(b)
        scale = scale_a if scale_a is not None else scale_b
        assert scale_a is None or scale_b is None or scale_a.dtype == scale_b.dtype
        w = w1 if w1 is not None else w2
        out = out1 if out1 is not None else out2
        assert (w1 is None) == (out1 is None) and (w2 is None) == (out2 is None)
        rc = self.lib.somi_add_scaled_rmsnorm(
            _ptr(residual), _ptr(a), ctypes.c_int(a_code), ctypes.c_int(a_splits),
            ctypes.c_longlong(a_stride), _ptr(scale_a), _ptr(b), ctypes.c_int(b_code),
            ctypes.c_int(b_splits), ctypes.c_longlong(b_stride), _ptr(scale_b),
            ctypes.c_int(_code(scale) if scale is not None else _F32), ctypes.c_float(mult),
            _ptr(extra), _ptr(w1), _ptr(w2), ctypes.c_int(_code(w) if w is not None else _F32),
            ctypes.c_float(eps), _ptr(out1), _ptr(out2),
            ctypes.c_int(_code(out) if out is not None else _F32), _ptr(rows), ctypes.c_int(n_out),
            ctypes.c_int(H), ctypes.c_int(0 if rows is not None else 1), self._stream())
        self._done(rc, "add_scaled_rmsnorm")
        if trace.active():
            n = n_out * H
            moved = n * 4 * (2 if rows is None else 1)
            for d, splits in ((a, a_splits), (b, b_splits)):
                if d is not None:
                    moved += splits * n * d.element_size()
            for o in (out1, out2):
                if o is not None:
                    moved += n * o.element_size()
            if extra is not None:
                moved += n * 4
            trace.note("add_scaled_rmsnorm", moved)

    def headnorm_rotary_store(self, qkv, positions, inv_freq, nq, nkv, hd, vd, rotary_dim, q_weight,
                              k_weight, eps, slot_map, kcache, vcache, magnitude: float = 1.0) -> None:
        """Rows of `qkv` hold nq query heads and nkv key heads of `hd` elements, then nkv value
        heads of `vd`.  Every query and key head passes an RMS norm over the head with
        `q_weight` / `k_weight` ([hd]; None: no norm); then entry i < rotary_dim / 2 and entry
        i + rotary_dim / 2 turn by position * inv_freq[i] (`inv_freq` float64), sine and cosine
        both multiplied by `magnitude`.  Queries are
        rewritten in place; keys and values go to their cache slots (`slot_map` None: nothing is
        stored)."""
        _check(positions, inv_freq, slot_map, kcache, vcache, q_weight, k_weight)
        if not (qkv.is_cuda and qkv.stride(1) == 1 and qkv.shape[1] >= (nq + nkv) * hd + nkv * vd):
            raise KernelError("headnorm_rotary_store takes a device tensor with contiguous rows")
        assert inv_freq.dtype == torch.float64 and inv_freq.numel() >= max(1, rotary_dim // 2)
        assert (q_weight is None) == (k_weight is None)
        page_size = 1
        if slot_map is not None:
            assert kcache.dtype == qkv.dtype and vcache.dtype == qkv.dtype
            assert kcache.shape[1] == nkv and kcache.shape[3] == hd and vcache.shape[3] == vd
            page_size = kcache.shape[2]
        rc = self.lib.somi_headnorm_rotary_store(
            _ptr(qkv), _code(qkv), ctypes.c_longlong(qkv.stride(0)), _ptr(positions), _ptr(inv_freq),
            ctypes.c_int(qkv.shape[0]), ctypes.c_int(nq), ctypes.c_int(nkv), ctypes.c_int(hd),
            ctypes.c_int(vd), ctypes.c_int(rotary_dim), _ptr(q_weight), _ptr(k_weight),
            ctypes.c_int(_code(q_weight) if q_weight is not None else _F32), ctypes.c_float(eps),
            ctypes.c_float(magnitude), _ptr(slot_map), _ptr(kcache), _ptr(vcache),
            ctypes.c_int(page_size), self._stream())
        self._done(rc, "headnorm_rotary_store")
        if trace.active():
            n = qkv.shape[0] * ((nq + nkv) * hd + nkv * vd)
            trace.note("headnorm_rotary_store", 2 * n * qkv.element_size())

    def check_matrix_state_geometry(self, heads: int, qk_heads: int, dk: int, dv: int) -> None:
        most = int(self.lib.somi_matrix_state_scan_max_key())
        if not (1 <= dk <= most and dv >= 1 and qk_heads >= 1 and heads % qk_heads == 0):
            raise KernelError(f"a matrix-state mixer with {heads} heads over {qk_heads} query/key "
                              f"heads of width {dk} is not supported (key width up to {most})")

    # a step in which some request has more rows than this has q, k and the decays made ready
    # once per row by a kernel of their own instead of once per group of state columns
    SCAN_PREPARE_ROWS = 16

    def matrix_state_scan(self, q, k, v, state, batch, y, heads, qk_heads, dk, dv, *,
                          act_silu=False, unit_eps=None, q_scale=1.0, beta=None, decay_logits=None,
                          dt_bias=None, a_log=None, decay=None, prepare=None) -> None:
        """Per request and head a float32 state S [dk, dv] in `state` [slots, heads, dv, dk] (a
        head's matrix column by column), continued over the request's rows of this step:
            S <- g * S;  u = v, or with `beta` u = sigmoid(beta) * (v - S^T k);  S <- S + k u^T;
            y = S^T q
        g is `decay` [heads], or per key channel exp(-exp(a_log) * softplus(decay_logits +
        dt_bias)) (`decay_logits` float32 [T, heads * dk], rows may lie further apart).  q, k
        ([T, qk_heads * dk]) and v ([T, heads * dv]) may be views of wider rows; `act_silu`: they
        pass SiLU as they are read; `unit_eps`: q and k are divided by sqrt(sum of squares + it);
        q is multiplied by `q_scale` either way.  y: float32 [T, heads * dv].  `prepare` (None: by the
        step's longest request) only chooses where q, k and g are computed; y is the same."""
        _check(state, y, dt_bias, a_log, decay)
        for t in (q, k, v, beta, decay_logits):
            if t is not None and not (t.is_cuda and t.stride(1) == 1):
                raise KernelError("matrix_state_scan takes device tensors with contiguous rows")
        assert q.dtype == k.dtype == v.dtype and (beta is None or beta.dtype == q.dtype)
        assert state.dtype == y.dtype == torch.float32 and tuple(state.shape[1:]) == (heads, dv, dk)
        assert decay_logits is None or decay_logits.dtype == torch.float32
        for t in (dt_bias, a_log, decay):
            assert t is None or t.dtype == torch.float32
        max_rows = int(getattr(batch, "max_q_len", 0) or 0)
        if prepare is None:
            prepare = max_rows > self.SCAN_PREPARE_ROWS
        act, unit, ready = (3 if act_silu else 0), (0 if unit_eps is None else 1), 0
        vb_code = _code(v)
        if prepare:
            T, n = q.shape[0], q.shape[0] * qk_heads * dk
            n_g = T * heads * dk if decay_logits is not None else 0
            buf = torch.empty(2 * n + n_g, dtype=torch.float32, device=q.device)
            qn, kn = buf[:n].view(T, -1), buf[n:2 * n].view(T, -1)
            gd = buf[2 * n:].view(T, -1) if n_g else None
            rc = self.lib.somi_matrix_state_prepare(
                _ptr(q), _ptr(k), _code(q), ctypes.c_longlong(q.stride(0)), ctypes.c_longlong(k.stride(0)),
                ctypes.c_int(act), ctypes.c_int(unit), ctypes.c_float(unit_eps or 0.0),
                ctypes.c_float(q_scale), _ptr(decay_logits),
                ctypes.c_longlong(decay_logits.stride(0) if decay_logits is not None else 0),
                _ptr(dt_bias), _ptr(a_log), _ptr(qn), _ptr(kn), _ptr(gd), ctypes.c_int(T),
                ctypes.c_int(heads), ctypes.c_int(qk_heads), ctypes.c_int(dk), self._stream())
            self._done(rc, "matrix_state_prepare")
            if trace.active():
                trace.note("matrix_state_prepare", 2 * n * (q.element_size() + 4) + 2 * n_g * 4)
            q, k, decay_logits = qn, kn, gd
            act, unit, ready, q_scale = act & 2, 0, 1, 1.0      # q is scaled already
        rc = self.lib.somi_matrix_state_scan(
            _ptr(q), _ptr(k), _ptr(v), _code(q), vb_code, ctypes.c_longlong(q.stride(0)),
            ctypes.c_longlong(k.stride(0)), ctypes.c_longlong(v.stride(0)),
            ctypes.c_int(act), ctypes.c_int(unit),
            ctypes.c_float(unit_eps or 0.0), ctypes.c_float(q_scale),
            ctypes.c_int(0 if beta is None else 1), _ptr(beta),
            ctypes.c_longlong(beta.stride(0) if beta is not None else 0), _ptr(decay_logits),
            ctypes.c_longlong(decay_logits.stride(0) if decay_logits is not None else 0),
            ctypes.c_int(ready),
            _ptr(dt_bias), _ptr(a_log), _ptr(decay), _ptr(state), _ptr(batch.cu_q),
            _ptr(batch.state_slot), _ptr(y), ctypes.c_int(batch.num_requests), ctypes.c_int(heads),
            ctypes.c_int(qk_heads), ctypes.c_int(dk), ctypes.c_int(dv),
            ctypes.c_int(max_rows), self._stream())
        self._done(rc, "matrix_state_scan")
        if trace.active():
            T = q.shape[0]
            moved = T * (2 * qk_heads * dk + heads * dv) * q.element_size() + T * heads * dv * 4 \
                + 2 * batch.num_requests * heads * dk * dv * 4
            if decay_logits is not None:
                moved += T * heads * dk * 4
            trace.note("matrix_state_scan", moved, (8.0 if beta is not None else 5.0) * T * heads * dk * dv,
                       detail="delta rule" if beta is not None else "decayed sum")

    def group_rmsnorm_gate(self, y, gate, weight, eps, groups, out, gate_act: str = "sigmoid") -> None:
        """out = rmsnorm over each of `groups` equal parts of y (float32), times weight (as long
        as a row, or as a part and then shared by the parts), times sigmoid(gate) where there is
        a gate ([T, C], rows may lie further apart); `gate_act` "silu": times silu(gate) instead."""
        _check(y, weight, out)
        if gate is not None and not (gate.is_cuda and gate.stride(1) == 1 and gate.shape == y.shape):
            raise KernelError("group_rmsnorm_gate takes a gate with contiguous rows")
        assert y.dtype == torch.float32
        C = y.shape[1]
        assert weight.numel() in (C, C // groups)
        rc = self.lib.somi_group_rmsnorm_gate(
            _ptr(y), _ptr(gate), ctypes.c_int(_code(gate) if gate is not None else _F32),
            ctypes.c_longlong(gate.stride(0) if gate is not None else 0), _ptr(weight), _code(weight),
            ctypes.c_int(weight.numel()), ctypes.c_float(eps), _ptr(out), _code(out),
            ctypes.c_int(y.shape[0]), ctypes.c_int(C), ctypes.c_int(groups),
            ctypes.c_int({"sigmoid": 0, "silu": 1}[gate_act]), self._stream())
        self._done(rc, "group_rmsnorm_gate")
        if trace.active():
            trace.note("group_rmsnorm_gate", y.numel() * (4 + out.element_size()
                                                          + (gate.element_size() if gate is not None else 0)))

    def rmsnorm_pair_mean(self, a, b, weight_a, weight_b, eps, out) -> None:
        """out = (rmsnorm(a) * weight_a + rmsnorm(b) * weight_b) / 2, float32 [T, H].  `a`, `b`:
        [T, H], or float32 [splits, T, H] partial sums that are added in order."""
        _check(a, b, weight_a, weight_b, out)
        assert out.dtype == torch.float32 and weight_a.dtype == weight_b.dtype
        T, H = out.shape

        def parts(d):
            assert tuple(d.shape[-2:]) == (T, H)
            if d.dim() == 3:
                assert d.dtype == torch.float32
                return _F32, d.shape[0], T * H
            return _code(d), 1, 0

        (a_code, a_splits, a_stride), (b_code, b_splits, b_stride) = parts(a), parts(b)
        rc = self.lib.somi_rmsnorm_pair_mean(
            _ptr(a), ctypes.c_int(a_code), ctypes.c_int(a_splits), ctypes.c_longlong(a_stride),
            _ptr(b), ctypes.c_int(b_code), ctypes.c_int(b_splits), ctypes.c_longlong(b_stride),
            _ptr(weight_a), _ptr(weight_b), _code(weight_a), ctypes.c_float(eps), _ptr(out),
            ctypes.c_int(T), ctypes.c_int(H), self._stream())
        self._done(rc, "rmsnorm_pair_mean")
        if trace.active():
            trace.note("rmsnorm_pair_mean", a.numel() * a.element_size() + b.numel() * b.element_size()
                       + out.numel() * 4)

    def relu2(self, x, out) -> None:
        """out = max(x, 0)^2, elementwise."""
        _check(x, out)
        assert x.dtype == out.dtype and x.shape == out.shape
        rc = self.lib.somi_relu2(_ptr(x), _ptr(out), _code(x), ctypes.c_longlong(x.numel()),
                                 self._stream())
        self._done(rc, "relu2")
        if trace.active():
            trace.note("relu2", 2 * x.numel() * x.element_size())

    def moe_router_select(self, logits, correction, count: int, keep: int, top: int,
                          over_chosen: bool = False):
        """logits float32 [T, n] -> (chosen int32 [T, top], weight float32 [T, top]): softmax over
        the n outputs; the choice is made on softmax + correction (None: the softmax) among the
        members of the `keep` best of `count` equal groups of neighbours (a group's score is its
        best member's; count <= 1: no groups); the weights are the chosen outputs' softmax.
        `over_chosen`: the `top` largest logits are chosen (no correction, no groups) and the
        weights are the softmax over the chosen logits only."""
        _check(logits, correction)
        assert logits.dtype == torch.float32 and (correction is None or correction.dtype == torch.float32)
        T, n = logits.shape
        chosen = torch.empty((T, top), dtype=torch.int32, device=logits.device)
        weight = torch.empty((T, top), dtype=torch.float32, device=logits.device)
        rc = self.lib.somi_moe_router_select(_ptr(logits), ctypes.c_longlong(logits.stride(0)),
                                             _ptr(correction), ctypes.c_int(T), ctypes.c_int(n),
                                             ctypes.c_int(count), ctypes.c_int(keep), ctypes.c_int(top),
                                             _ptr(chosen), _ptr(weight),
                                             ctypes.c_int(1 if over_chosen else 0), self._stream())
        self._done(rc, "moe_router_select")
        if trace.active():
            trace.note("moe_router_select", T * (n * 4 + top * 8))
        return chosen, weight

    def moe_combine_weighted(self, y, place, table, weight, x, num_experts: int) -> torch.Tensor:
        """out[t] = sum_k weight[t, k] * (y[row(t * top + k)] if table[t, k] < num_experts else
        x[t]); float32 [T, H].  `place`: the row of every entry where y's rows are in the grouped
        order (None: row = entry)."""
        _check(y, place, table, weight, x)
        T, top = table.shape
        H = x.shape[1]
        assert y.shape[1] == H and weight.dtype == torch.float32 and table.dtype == torch.int32
        out = torch.empty((T, H), dtype=torch.float32, device=x.device)
        rc = self.lib.somi_moe_combine_weighted(_ptr(y), _code(y), _ptr(place), _ptr(table), _ptr(weight),
                                                _ptr(x), _code(x), ctypes.c_int(num_experts),
                                                ctypes.c_int(top), ctypes.c_int(T), ctypes.c_int(H),
                                                _ptr(out), self._stream())
        self._done(rc, "moe_combine_weighted")
        if trace.active():
            trace.note("moe_combine_weighted", T * top * H * y.element_size() + T * H * (4 + x.element_size()))
        return out

    def silu_mul(self, gu: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
        """out = silu(gate) * up; gate/up are the two halves of `gu`'s rows, or alternate."""
        _check(gu, out)
        rc = self.lib.somi_silu_mul(_ptr(gu), _ptr(out), _code(gu), ctypes.c_longlong(gu.shape[0]),
                                    ctypes.c_int(out.shape[1]), ctypes.c_int(1 if interleaved else 0),
                                    self._stream())
        self._done(rc, "silu_mul")
        if trace.active():
            trace.note("silu_mul", (gu.numel() + out.numel()) * gu.element_size())

    # ------------------------------------------------------- tcgen05 matrix product
    GEMM_BF16, GEMM_F32, GEMM_PARTIAL_F32, GEMM_SWIGLU, GEMM_XIELU_SIDE = 0, 1, 2, 3, 4

    def skinny_splits(self, M: int, N: int, K: int) -> int:
        """How many ranges of K to run side by side: CTAs for about one and a half per SM, at
        least three K blocks each, at most eight (the consumer reads every partial sum: 4 *
        splits * M * N bytes, written and read back), and partial sums that stay below a quarter
        of the weight's own bytes.  Measured with the consumer (norm or rotary kernel) behind
        each product in CUDA graphs, 1 and 8 tokens: more splits than this cost the 0.5B shape's
        down projection 1.2 µs (16 -> 8) and the 7B shape's output projection 0.4 µs (10 -> 8);
        past two CTAs per SM a product takes a third longer."""
        tiles = -(-N // 128)
        k_blocks = -(-K // 64)
        return max(1, min(224 // tiles, k_blocks // 3, K // (16 * M), 8))

    def skinny_supported(self, M: int, N: int, K: int, dtype) -> bool:
        """Whether the tensor-memory kernel takes x[M, K] @ w[N, K]^T (few tokens, bfloat16)."""
        if not (self.use_skinny_gemm and dtype == torch.bfloat16
                and 1 <= M <= self.skinny_max_tokens and K % 8 == 0 and N >= 1):
            return False
        # measured (CUDA graphs of back-to-back products with their consumers, and whole decode
        # steps at batch 32 and 64): above 16 tokens this kernel wins only where a CTA streams a
        # long K range, of a large matrix or of one that is several times as long as it is wide
        # (the 0.5B shape's down projection at 24-64 tokens: 7.8-9.5 µs against the library's
        # 11.4-11.7); short K (few stages per CTA) and small matrices go to the library
        return M <= 16 or (K >= 2048 and (N * K >= (32 << 20) or K >= 4 * N))

    def _gemm_map(self, t: torch.Tensor, box_rows: int) -> int:
        key = (t.data_ptr(), t.shape[0], t.shape[1], box_rows)
        entry = self._gemm_maps.get(key)
        if entry is None:
            if len(self._gemm_maps) > 8192:
                self._gemm_maps.clear()
            raw = (ctypes.c_ubyte * 256)()
            addr = (ctypes.addressof(raw) + 127) & ~127
            rc = self.lib.somi_make_gemm_tensor_map(ctypes.c_void_p(addr), _ptr(t),
                                                    ctypes.c_longlong(t.shape[0]),
                                                    ctypes.c_longlong(t.shape[1]),
                                                    ctypes.c_int(box_rows))
            if rc != 0:
                raise KernelError(f"could not encode a tensor map over a {tuple(t.shape)} matrix (code {rc})")
            entry = (raw, addr)
            self._gemm_maps[key] = entry
        return entry[1]

    def skinny_gemm(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
                    mode: int = 0, splits: int = 1, deep_ring: bool = False,
                    act: torch.Tensor | None = None, n_act: int = 0):
        """x[M, K] @ w[N, K]^T on tcgen05 tensor cores for M <= 64.

        mode GEMM_BF16 -> bf16 [M, N] (+ bias); GEMM_F32 -> float32 [M, N];
        GEMM_PARTIAL_F32 -> float32 [splits', M, N] partial sums over ranges of K (bias in the
        first); GEMM_SWIGLU -> bf16 [M, N / 2] = silu(even rows) * odd rows of w;
        GEMM_XIELU_SIDE -> (bf16 [M, n_act] = xIELU of the first n_act features with the two
        numbers of `act` (float32), bf16 [M, N - n_act] = the other features), bias added to both.
        """
        _check(x, w, bias)
        M, K = x.shape
        N = w.shape[0]
        assert w.shape[1] == K and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
        box = 16 if M <= 16 else (32 if M <= 32 else 64)
        if mode == self.GEMM_PARTIAL_F32:
            splits = int(self.lib.somi_skinny_gemm_splits(ctypes.c_int(K), ctypes.c_int(splits)))
            out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        elif mode == self.GEMM_F32:
            out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        elif mode == self.GEMM_SWIGLU:
            out = torch.empty((M, N // 2), dtype=torch.bfloat16, device=x.device)
        elif mode == self.GEMM_XIELU_SIDE:
            _check(act)
            assert act is not None and act.dtype == torch.float32 and act.numel() == 2
            assert 0 <= n_act <= N
            out = torch.empty((M, n_act), dtype=torch.bfloat16, device=x.device)
            out2 = torch.empty((M, N - n_act), dtype=torch.bfloat16, device=x.device)
        else:
            out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
        # few CTAs: one per SM with the whole shared memory as an 8-stage ring (a CTA's stream
        # is bound by the bytes it keeps in flight); many CTAs: two per SM with 4 stages each
        ctas = -(-N // 128) * (splits if mode == self.GEMM_PARTIAL_F32 else 1)
        deep_ring = deep_ring or ctas <= 148
        if mode == self.GEMM_XIELU_SIDE:
            rc = self.lib.somi_skinny_gemm_act(
                ctypes.c_void_p(self._gemm_map(w, 128)), ctypes.c_void_p(self._gemm_map(x, box)),
                ctypes.c_int(box), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                ctypes.c_int(1), ctypes.c_int(mode), _ptr(bias),
                _code(bias) if bias is not None else _F32, _ptr(out), _ptr(out2),
                ctypes.c_int(n_act), _ptr(act), ctypes.c_int(1 if deep_ring else 0), self._stream())
        else:
            rc = self.lib.somi_skinny_gemm(
                ctypes.c_void_p(self._gemm_map(w, 128)), ctypes.c_void_p(self._gemm_map(x, box)),
                ctypes.c_int(box), ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K),
                ctypes.c_int(splits), ctypes.c_int(mode), _ptr(bias),
                _code(bias) if bias is not None else _F32, _ptr(out),
                ctypes.c_int(1 if deep_ring else 0), self._stream())
        self._done(rc, "skinny_gemm")
        if trace.active():
            trace.note("skinny_gemm", (N * K + M * K) * 2 + out.numel() * out.element_size(),
                       2.0 * M * N * K, detail=f"M={M} N={N} K={K} mode={mode}")
        if mode == self.GEMM_XIELU_SIDE:
            return out, out2
        return out

    def gemm_f32(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """x[M, K] @ w[N, K]^T (+ bias) in float32 FMAs, each output summed over K in ascending
        order (the float32 path's product; the library's is not used there)."""
        _check(x, w, bias)
        M, K = x.shape
        N = w.shape[0]
        if not (x.dtype == w.dtype == torch.float32 and w.shape[1] == K
                and (bias is None or (bias.dtype == torch.float32 and bias.numel() == N))):
            raise KernelError("gemm_f32 takes float32 x[M, K], w[N, K] and bias[N]")
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        rc = self.lib.somi_gemm_f32(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), ctypes.c_int(M),
                                    ctypes.c_int(N), ctypes.c_int(K), self._stream())
        self._done(rc, "gemm_f32")
        if trace.active():
            trace.note("gemm_f32", (N * K + M * K + M * N) * 4, 2.0 * M * N * K, detail=f"M={M} N={N} K={K}")
        return out

    def sample(self, logits, temperature, top_k, top_p, penalty, seed, counter, hist_off,
               hist_tok, out) -> None:
        """seed: int32 view of uint64 pairs [2 * rows]; counter: int32 view of uint32 [rows]."""
        _check(logits, temperature, top_k, top_p, penalty, seed, counter, hist_off, hist_tok, out)
        assert logits.dtype == torch.float32 and out.dtype == torch.int32
        assert seed.data_ptr() % 8 == 0
        rc = self.lib.somi_sample(_ptr(logits), ctypes.c_int(logits.shape[0]),
                                  ctypes.c_int(logits.shape[1]), _ptr(temperature), _ptr(top_k),
                                  _ptr(top_p), _ptr(penalty), _ptr(seed), _ptr(counter),
                                  _ptr(hist_off), _ptr(hist_tok), _ptr(out), self._stream())
        self._done(rc, "sample")
        if trace.active():
            trace.note("sample", logits.numel() * 4)

    def uniform(self, seed: int, counter: int) -> float:
        """The uniform number in [0, 1) that row (seed, counter) draws (host evaluation)."""
        self.lib.somi_sample_uniform.restype = ctypes.c_float
        return float(self.lib.somi_sample_uniform(ctypes.c_ulonglong(seed), ctypes.c_uint(counter)))


_OPS: CudaOps | None = None


def cuda_ops() -> CudaOps:
    """The process-wide kernel table (built and loaded at first use)."""
    global _OPS
    if _OPS is None:
        _OPS = CudaOps()
    return _OPS
