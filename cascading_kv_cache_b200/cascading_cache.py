"""CascadingKVCache: the reference's cache object with its state in HBM and every
mutation done by the sm_100a kernels of libckv_b200.so.

Interface mirrors cascade/models/cascading_cache.py:1031-1348 of the reference
(constructor arguments, ``update``, ``get_vals``, ``reset``, ``get_seq_length``,
``get_max_length``, indexing/iteration, the per-layer state lists, ``beta``).

Memory layout differences (values are identical to the reference's):

* ``mask``, ``sink_mask``, ``pos``, ``sink_pos``, ``stored_tokens``,
  ``start_indices`` and ``stored_sinks`` depend only on how many tokens a layer
  has seen, never on the lane (batch, kv head).  They are stored once and
  exposed as stride-0 expanded views with the reference's shapes
  (``[B, H, ...]``), so indexing code keeps working while a decode step writes
  ``S`` position words instead of ``B*H*S``.
* ``seen_tokens_by_layer`` lives on the device and is advanced by the kernels;
  a host-side integer mirror removes the host synchronisations the reference
  performs in ``get_vals`` (:1282) and in the attention forward
  (cascade_attention.py:114).
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import List, Optional, Union

import torch
from transformers.cache_utils import Cache

from . import _lib

CASCADE_FUNCS = ("pow2", "pow2-1", "pow2-1-4", "pow2-2-4", "pow2-3-4", "1-then-2", "pow3", "pow4", "iplus1")


def cascade_every_n(cascade_func: str, cascades: int) -> List[int]:
    """Admission stride of each cascade (reference init_cache, cascading_cache.py:1201-1244)."""
    c, n = cascades, cascades // 4
    table = {
        "pow2": lambda: [2 ** i for i in range(c)],
        "pow2-1": lambda: [1] * (c - 1) + [2 ** i for i in range(c - 1, c)],
        "pow2-1-4": lambda: [1] * (3 * n) + [2 ** i for i in range(3 * n, c)],
        "pow2-2-4": lambda: [1] * (2 * n) + [2 ** i for i in range(2 * n, c)],
        "pow2-3-4": lambda: [1] * n + [2 ** i for i in range(n, c)],
        "1-then-2": lambda: [1] + [2] * (c - 1),
        "pow3": lambda: [3 ** i for i in range(c)],
        "pow4": lambda: [4 ** i for i in range(c)],
        "iplus1": lambda: [i + 1 for i in range(c)],
    }
    if cascade_func not in table:
        raise ValueError(f"unknown cascade func: {cascade_func}")
    return table[cascade_func]()


def _one_row(t: torch.Tensor, lead_dims: int):
    """Pointer source for a lane-invariant state tensor given with the reference's ``[B, H, ...]`` shape.
    Returns ``(row, broadcast)``: ``row`` is the single row the kernels read and write; ``broadcast`` says
    whether the tensor really stores one row per lane, in which case the caller copies the row back to
    every lane after the launch (the views this package's cache exposes have stride 0 and need no copy)."""
    row = t[(0,) * lead_dims]
    shared = all(t.stride(i) == 0 or t.size(i) == 1 for i in range(lead_dims))
    return row, not shared


def sink_cache(k, v, s, sink_k, sink_v, sink_mask, sink_pos, cache_k, cache_v, cache_s, mask, pos, og_pos,
               do_cache, do_cache_every_n, stored_tokens, start_indices, stored_sinks, num_sink, window_size,
               real_token_idx, max_seq_len, eager_fill, BENCHMARK: bool = False):
    """The reference's functional update, ``sink_cache(...)`` (cascade/models/cascading_cache.py:962-1028),
    with the same 23 positional arguments, served by one ``ckv_cascade_update`` call.

    Tensors keep the reference's shapes: ``k, v [N,H,K,D]``, ``s [N,>=H,K]``, sinks ``[N,H,NS,D]``, cache
    ``[N,H,S,D]``, ``cache_s [N,H,S]``, ``mask/pos/og_pos [N,H,S]``, ``sink_mask/sink_pos [N,H,NS]``, counters
    ``[N,H,C]`` / ``[N,H]``; ``real_token_idx`` is the device scalar holding the tokens seen so far and is
    left as it is (the reference's caller advances it, :1346).  ``do_cache`` is accepted and unused, as in
    the reference kernel.  Lane-invariant tensors (masks, positions, counters) may be the stride-0 views of
    this package's cache or real per-lane tensors; the latter are updated on lane (0, 0) and copied to the
    other lanes.  With ``BENCHMARK`` the launch is timed with CUDA events and the time printed (:986-1026).
    Returns ``(k, v)``."""
    N, H, K, D = k.shape
    if v.shape != k.shape:
        raise ValueError("k and v must have the same shape")
    if k.device.type != "cuda":
        raise RuntimeError("sink_cache runs on a CUDA device only (there is no CPU path)")
    if k.dtype not in _lib.DTYPE_CODE:
        raise ValueError(f"unsupported dtype {k.dtype}")
    for name, t in (("cache_k", cache_k), ("cache_v", cache_v), ("cache_s", cache_s), ("og_pos", og_pos)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
    for name, t in (("sink_k", sink_k), ("sink_v", sink_v)):
        if t.numel() and not (t.stride(3) == 1 and t.stride(2) == D and t.stride(1) == num_sink * D
                               and t.stride(0) == H * num_sink * D):
            raise ValueError(f"{name} must be laid out as [N, H, {num_sink}, {D}] rows")
    C = stored_tokens.size(-1)
    if max_seq_len != C * window_size or cache_k.size(2) != max_seq_len:
        raise ValueError("max_seq_len must equal cascades * window_size and the cache length")
    lib = _lib.load()
    dt, dev = k.dtype, k.device
    conv = lambda t: t if (t.dtype == dt and t.device == dev) else t.to(device=dev, dtype=dt)
    k2, v2 = conv(k), conv(v)
    rows16 = lambda t: (t.stride(3) == 1 and t.data_ptr() % 16 == 0
                        and all((t.stride(i) * t.element_size()) % 16 == 0 for i in range(3)))
    if not (rows16(k2) and rows16(v2) and k2.stride() == v2.stride()):
        k2, v2 = k2.contiguous(), v2.contiguous()
    s_ptr, ss = None, (0, 0, 0)
    if s is not None:
        s2 = conv(s)
        s_ptr, ss = s2.data_ptr(), s2.stride()
    m8 = mask.view(torch.uint8) if mask.dtype == torch.bool else mask
    sm8 = sink_mask.view(torch.uint8) if sink_mask.dtype == torch.bool else sink_mask
    shared = {}
    for name, t, lead in (("mask", m8, 2), ("sink_mask", sm8, 2), ("pos", pos, 2), ("sink_pos", sink_pos, 2),
                          ("stored_tokens", stored_tokens, 2), ("start_indices", start_indices, 2),
                          ("stored_sinks", stored_sinks, 2)):
        shared[name] = (t,) + _one_row(t, lead)
    seen = real_token_idx.reshape(-1)[:1].clone()     # the kernel advances its counter; the caller's stays
    every = do_cache_every_n.to(device=dev, dtype=torch.long).contiguous()
    cfg = _lib.CkvConfig(batch=N, kv_heads=H, q_heads=H, head_dim=D, num_sinks=int(num_sink), window=int(window_size),
                         cascades=C, dtype=_lib.DTYPE_CODE[dt], eager_fill=int(bool(eager_fill)), head_reduction=0,
                         homogeneous_heads=0, admission=_lib.CKV_ADMIT["ema"], beta=1.0)
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    st = _lib.CkvLayerState(
        key_cache=p(cache_k), value_cache=p(cache_v), score_cache=p(cache_s), sink_keys=p(sink_k),
        sink_values=p(sink_v), mask=p(shared["mask"][1]), sink_mask=p(shared["sink_mask"][1]),
        pos=p(shared["pos"][1]), og_pos=p(og_pos), sink_pos=p(shared["sink_pos"][1]),
        stored_tokens=p(shared["stored_tokens"][1]), start_indices=p(shared["start_indices"][1]),
        stored_sinks=p(shared["stored_sinks"][1]), seen_tokens=p(seen), every_n=p(every))
    ws, ws_ptr, ws_bytes = None, None, 0
    if K >= 2:
        ws_bytes = lib.ckv_update_workspace_bytes(ctypes.byref(cfg), K)
        ws = torch.empty(ws_bytes + 256, device=dev, dtype=torch.uint8)
        ws_ptr = (ws.data_ptr() + 255) & ~255
    if BENCHMARK:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
    with torch.cuda.device(dev):
        rc = lib.ckv_cascade_update(ctypes.byref(cfg), ctypes.byref(st), k2.data_ptr(), v2.data_ptr(), k2.stride(0),
                                    k2.stride(1), k2.stride(2), s_ptr, ss[0], ss[1], ss[2], K, ws_ptr, ws_bytes,
                                    _lib.current_stream_ptr(dev))
    _lib.check(rc, "ckv_cascade_update")
    for name, (t, row, broadcast) in shared.items():
        if broadcast:
            t.copy_(row.expand_as(t))
    if BENCHMARK:
        ev1.record()
        torch.cuda.synchronize()
        print(ev0.elapsed_time(ev1))
    return k, v


class CascadingKVCache(Cache):
    # transformers >= 5 declares these as read-only properties on Cache; the
    # reference assigns them as plain attributes, so shadow them here.
    max_batch_size = None
    max_cache_len = None
    is_compileable = False
    is_initialized = True
    is_sliding = None

    def __init__(
        self,
        window_length: Union[int, List[int]] = 8,
        num_sink_tokens: int = 4,
        max_batch_size: int = 1,
        heads: int = 16,
        dim: int = 128,
        max_seq_len: Union[int, List[int]] = 32,
        device: torch.device = "cpu",
        dtype: torch.dtype = torch.float16,
        cascade_func: str = "pow2",
        head_reduction: str = "mean",
        layers: int = 32,
        eager_fill: bool = True,
        verbose: bool = True,
        admission: str = "ema",
    ) -> None:
        # Cache.__init__ of transformers >= 5 wants layer objects; this cache owns its tensors.
        if isinstance(max_seq_len, int) != isinstance(window_length, int):
            raise ValueError(
                f"max_seq_len must be same type as window length: {type(max_seq_len)=} {type(window_length)=}")
        if isinstance(max_seq_len, int):
            max_seq_len = [max_seq_len for _ in range(layers)]
        if isinstance(window_length, int):
            window_length = [window_length for _ in range(layers)]
        if dtype not in _lib.DTYPE_CODE:
            raise ValueError(f"unsupported cache dtype {dtype}")
        if head_reduction not in _lib.CKV_REDUCE:
            raise ValueError(f"unknown head reduction: {head_reduction}")
        if admission not in _lib.CKV_ADMIT:
            raise ValueError(f"unknown admission rule: {admission}")
        if cascade_func not in CASCADE_FUNCS:
            raise ValueError(f"unknown cascade func: {cascade_func}")
        if not all((max_seq_len[l] % window_length[l]) == 0 for l in range(layers)):
            raise ValueError(
                f"window length must evenly divide max seq len: {window_length=} {max_seq_len=}")
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("CascadingKVCache lives in GPU memory: the device must be a CUDA device "
                               "(there is no CPU path)")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())

        self.verbose = verbose
        self.max_seq_len = max_seq_len
        self.max_batch_size = max_batch_size
        self.heads = heads
        self.dim = dim
        self.device = device
        self.dtype = dtype
        self.window_length = window_length
        self.num_sink_tokens = num_sink_tokens
        self.cascade_func = cascade_func
        self.head_reduction = head_reduction
        self.layers = layers
        self.eager_fill = eager_fill
        self.admission = admission
        self.bh = max_batch_size * heads

        self.cascades = [max_seq_len[l] // window_length[l] for l in range(layers)]
        self._seen_tokens = 0
        self._lib = _lib.load()
        self.init_cache(self.device)

    def __repr__(self):
        return f"{self.max_seq_len=}, {self.cascades=} {self.max_batch_size=}, {self.layers=} {self.heads=}"

    def __getitem__(self, layer_idx: int):
        return self.get_vals(layer_idx)

    def __iter__(self):
        for layer_idx in range(len(self)):
            yield self.get_vals(layer_idx)

    def __len__(self):
        return self.layers

    # ------------------------------------------------------------------ state
    def init_cache(self, device):
        L, B, H, D = self.layers, self.max_batch_size, self.heads, self.dim
        NS, dt = self.num_sink_tokens, self.dtype
        if self.verbose:
            print(f"INIT CLEAN CASCADE CACHE {self.cascade_func=}")
        z = lambda *shape, dtype=dt: torch.zeros(*shape, device=device, dtype=dtype)

        self._seen_tokens = 0
        self._seen_host = [0 for _ in range(L)]
        self.seen_tokens_by_layer = z(L, dtype=torch.long)
        # original submission used 0.9999; the reference later raised it (cascading_cache.py:1246-1247)
        self.beta = 0.9999999

        self.do_cache = [torch.ones(self.cascades[l], device=device, dtype=torch.bool) for l in range(L)]
        self.do_cache_every_n = [
            torch.tensor(cascade_every_n(self.cascade_func, self.cascades[l]), device=device, dtype=torch.long)
            for l in range(L)]

        # lane-invariant state: one row, exposed with the reference's shapes through expand()
        self._stored_tokens = [z(self.cascades[l], dtype=torch.long) for l in range(L)]
        self._start_indices = [z(self.cascades[l], dtype=torch.long) for l in range(L)]
        self._stored_sinks = [z(1, dtype=torch.long) for _ in range(L)]
        self._pos = [z(self.max_seq_len[l], dtype=torch.long) for l in range(L)]
        self._sink_pos = [z(max(NS, 1), dtype=torch.long)[:NS] for _ in range(L)]
        self._mask = [torch.ones(self.max_seq_len[l], device=device, dtype=torch.bool) for l in range(L)]
        self._sink_mask = [torch.ones(max(NS, 1), device=device, dtype=torch.bool)[:NS] for _ in range(L)]

        self.stored_tokens = [t.view(1, 1, -1).expand(B, H, -1) for t in self._stored_tokens]
        self.start_indices = [t.view(1, 1, -1).expand(B, H, -1) for t in self._start_indices]
        self.stored_sinks = [t.view(1, 1).expand(B, H) for t in self._stored_sinks]
        self.pos = [t.view(1, 1, -1).expand(B, H, -1) for t in self._pos]
        self.sink_pos = [t.view(1, 1, -1).expand(B, H, -1) for t in self._sink_pos]
        self.mask = [t.view(1, 1, -1).expand(B, H, -1) for t in self._mask]
        self.sink_mask = [t.view(1, 1, -1).expand(B, H, -1) for t in self._sink_mask]

        # per-lane state
        self.og_pos = [z(B, H, self.max_seq_len[l], dtype=torch.long) for l in range(L)]
        self.key_cache = [z(B, H, self.max_seq_len[l], D) for l in range(L)]
        self.value_cache = [z(B, H, self.max_seq_len[l], D) for l in range(L)]
        self.score_cache = [z(B, H, self.max_seq_len[l]) for l in range(L)]
        self.sink_keys = [z(B, H, max(NS, 1), D)[:, :, :NS] for _ in range(L)]
        self.sink_values = [z(B, H, max(NS, 1), D)[:, :, :NS] for _ in range(L)]

        self._workspace = None
        self.force_serial_update = False   # tests: take the one-warp-per-lane update also for chunks
        self._rope_tables = {}
        self._ema_weights = {}
        self._cfg_cache = {}
        self._state_cache = [None for _ in range(L)]
        # host mirror of the lane-invariant counters (sinks, stored[C], start[C]) and the token count
        # they are valid for; None = unknown, read from the device on first use
        self._host_counters = [((0, [0] * self.cascades[l], [0] * self.cascades[l]), 0) for l in range(L)]

    def reset(self, verbose=True):
        if verbose and self.verbose:
            print(f"RESET CASCADE CACHE {self.cascade_func=}")
        self._seen_tokens = 0
        self._seen_host = [0 for _ in range(self.layers)]
        self._host_counters = [((0, [0] * self.cascades[l], [0] * self.cascades[l]), 0) for l in range(self.layers)]
        self.seen_tokens_by_layer.zero_()
        for group in (self._stored_tokens, self._start_indices, self._stored_sinks, self._pos, self._sink_pos,
                      self.og_pos, self.key_cache, self.value_cache, self.score_cache, self.sink_keys,
                      self.sink_values):
            for t in group:
                t.zero_()
        for t in self.do_cache:
            t.fill_(True)
        for t in self._mask + self._sink_mask:
            t.fill_(True)

    # ------------------------------------------------------------- ABI helpers
    def ckv_config(self, layer_idx: int, q_heads: Optional[int] = None, homogeneous_heads: bool = False,
                   head_reduction: Optional[str] = None, admission: Optional[str] = None) -> _lib.CkvConfig:
        q_heads = self.heads if q_heads is None else q_heads
        key = (layer_idx, q_heads, homogeneous_heads, head_reduction or self.head_reduction,
               admission or self.admission, self.beta, self.eager_fill)
        cfg = self._cfg_cache.get(key)
        if cfg is None:
            cfg = _lib.CkvConfig(
                batch=self.max_batch_size, kv_heads=self.heads, q_heads=q_heads, head_dim=self.dim,
                num_sinks=self.num_sink_tokens, window=self.window_length[layer_idx],
                cascades=self.cascades[layer_idx], dtype=_lib.DTYPE_CODE[self.dtype],
                eager_fill=int(self.eager_fill), head_reduction=_lib.CKV_REDUCE[key[3]],
                homogeneous_heads=int(homogeneous_heads), admission=_lib.CKV_ADMIT[key[4]], beta=float(self.beta))
            cfg.ref = ctypes.byref(cfg)     # made once: a decode call then builds no ctypes objects
            cfg.ws_bytes = {}
            self._cfg_cache[key] = cfg
        return cfg

    def attention_workspace_bytes(self, cfg: _lib.CkvConfig, n_tokens: int, flags: int) -> int:
        """``ckv_attention_workspace_bytes_for`` with the answer remembered per (config, tokens, flags)."""
        n = cfg.ws_bytes.get((n_tokens, flags))
        if n is None:
            n = cfg.ws_bytes[(n_tokens, flags)] = self._lib.ckv_attention_workspace_bytes_for(cfg.ref, n_tokens, flags)
        return n

    def ckv_state(self, layer_idx: int) -> _lib.CkvLayerState:
        """The layer's device pointers as the ABI struct, built once per layer and reused while the
        tensors it points at are the same objects."""
        l = layer_idx
        # score_cache[l] may have been re-assigned from Python (the reference's attention does); re-read pointers
        sc = self.score_cache[l]
        cached = self._state_cache[l]
        if cached is not None and cached[1] is sc and cached[2] is self.key_cache[l]:
            return cached[0]
        if (sc.dtype != self.dtype or not sc.is_contiguous() or sc.device != self.device
                or tuple(sc.shape) != (self.max_batch_size, self.heads, self.max_seq_len[l])):
            sc = sc.to(device=self.device, dtype=self.dtype).expand(
                self.max_batch_size, self.heads, self.max_seq_len[l]).contiguous()
            self.score_cache[l] = sc
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        st = _lib.CkvLayerState(
            key_cache=p(self.key_cache[l]), value_cache=p(self.value_cache[l]), score_cache=p(sc),
            sink_keys=p(self.sink_keys[l]), sink_values=p(self.sink_values[l]),
            mask=p(self._mask[l]), sink_mask=p(self._sink_mask[l]), pos=p(self._pos[l]), og_pos=p(self.og_pos[l]),
            sink_pos=p(self._sink_pos[l]), stored_tokens=p(self._stored_tokens[l]),
            start_indices=p(self._start_indices[l]), stored_sinks=p(self._stored_sinks[l]),
            seen_tokens=ctypes.c_void_p(self.seen_tokens_by_layer.data_ptr() + 8 * l),
            every_n=p(self.do_cache_every_n[l]))
        st.ref = ctypes.byref(st)
        self._state_cache[l] = (st, sc, self.key_cache[l])
        return st

    def device_guard(self):
        """Context that makes the cache's device current: the library launches on the calling
        thread's current device.  Free when it already is."""
        if torch.cuda.current_device() == self.device.index:
            return contextlib.nullcontext()
        return torch.cuda.device(self.device)

    def workspace(self, nbytes: int) -> torch.Tensor:
        if self._workspace is None or self._workspace.numel() < nbytes:
            self._workspace = torch.empty(nbytes + 256, device=self.device, dtype=torch.uint8)
            self._workspace[:512].zero_()     # the status word reads 0 until an attention call writes it
        return self._workspace

    def workspace_bytes(self) -> int:
        return 0 if self._workspace is None else self._workspace.numel() - 256

    def workspace_ptr(self) -> int:
        return (self._workspace.data_ptr() + 255) & ~255

    def kernel_status(self) -> int:
        """Status word of the last attention call (synchronises): 0 unless a bounded wait inside a
        kernel ran out, in which case that call's results are invalid."""
        if self._workspace is None:
            return 0
        status = ctypes.c_int32(0)
        with self.device_guard():
            _lib.check(self._lib.ckv_read_status(self.workspace_ptr(), ctypes.byref(status)), "ckv_read_status")
        return int(status.value)

    def rope_table(self, theta: float, rows: int) -> torch.Tensor:
        """[rows, D] table in the cache dtype: cos | sin of position * inv_freq, computed like
        LlamaRotaryEmbedding.forward (fp32 angles, fp32 cos/sin, cast)."""
        key = float(theta)
        tab = self._rope_tables.get(key)
        if tab is None or tab.size(0) < rows:
            rows = max(rows, (tab.size(0) * 2) if tab is not None else 0)
            inv_freq = 1.0 / (theta ** (torch.arange(0, self.dim, 2, dtype=torch.int64).float() / self.dim))
            freqs = torch.arange(rows, dtype=torch.int64).float()[:, None] * inv_freq[None, :]
            tab = torch.cat((freqs.cos(), freqs.sin()), dim=-1).to(self.dtype).to(self.device).contiguous()
            self._rope_tables[key] = tab
        return tab

    def ema_weights(self, n_tokens: int):
        """EMA weight vectors of one attention call, computed with the same torch expressions as the
        reference (cascade_attention.py:272-276 and :316-317)."""
        key = (n_tokens, float(self.beta))
        w = self._ema_weights.get(key)
        if w is None:
            beta = self.beta
            w_cache = ((1 - beta) * beta ** torch.arange(n_tokens).flip(dims=(0,))).to(torch.float32)
            w_new = (1 - beta) * beta ** torch.arange(n_tokens, dtype=self.dtype)
            w = (w_cache.to(self.device).contiguous(), w_new.to(self.device).contiguous())
            if len(self._ema_weights) > 64:
                self._ema_weights.clear()
            self._ema_weights[key] = w
        return w

    # --------------------------------------------------------------- interface
    def invalidate_host_counters(self, layer_idx: Optional[int] = None):
        """Call after writing the counter tensors directly (tests, synthetic set-ups): the host
        mirror is re-read from the device the next time it is needed."""
        for l in (range(self.layers) if layer_idx is None else [layer_idx]):
            self._host_counters[l] = None

    def host_counters(self, layer_idx: int):
        """(stored_sinks, stored_tokens[C], start_indices[C]) of a layer without touching the device:
        the counters depend only on how many tokens the layer has seen, so a host copy is advanced
        by the same state machine the kernels run (cascading_cache.py:381-726 of the reference, the
        branches that never look at scores)."""
        l = layer_idx
        C = self.cascades[l]
        entry = self._host_counters[l]
        if entry is None:       # written from outside: one device read, then tracked on the host again
            sinks = int(self._stored_sinks[l].item())
            entry = ((sinks, self._stored_tokens[l].tolist(), self._start_indices[l].tolist()), self._seen_host[l])
        (sinks, stored, start), at = entry
        todo = self._seen_host[l] - at
        if todo > 0:
            arr = ctypes.c_int64 * C
            c_stored, c_start, c_sinks = arr(*stored), arr(*start), ctypes.c_int64(sinks)
            every = arr(*cascade_every_n(self.cascade_func, C))
            cfg = self.ckv_config(l)
            _lib.check(self._lib.ckv_advance_counters_host(ctypes.byref(cfg), every, at, todo, c_stored, c_start,
                                                           ctypes.byref(c_sinks)), "ckv_advance_counters_host")
            sinks, stored, start = int(c_sinks.value), list(c_stored), list(c_start)
        self._host_counters[l] = ((sinks, stored, start), self._seen_host[l])
        return sinks, stored, start

    def get_seq_length(self, layer_idx: Optional[int] = 0, cascade_idx: Optional[int] = -1) -> int:
        """Tokens held by the layer (sinks + every cascade), reference cascading_cache.py:1129-1132,
        from the host mirror of the counters: no device synchronisation."""
        sinks, stored, _ = self.host_counters(layer_idx)
        return sinks + sum(stored)

    def get_max_length(self) -> Optional[int]:
        return self.max_seq_len[0]

    def get_max_cache_shape(self, layer_idx: int = 0) -> int:
        return self.max_seq_len[layer_idx]

    def seen_tokens_host(self, layer_idx: int) -> int:
        """Tokens this layer has seen, from the host mirror (no device synchronisation)."""
        return self._seen_host[layer_idx]

    def get_vals(self, layer_idx: int):
        """The reference's 9-tuple (cascading_cache.py:1278-1295).  The +num_sink_tokens shift of the
        cache positions is decided from the host mirror of the token counter."""
        pos_shift = self.num_sink_tokens if self._seen_host[layer_idx] > self.num_sink_tokens else 0
        return (
            self.sink_keys[layer_idx],
            self.sink_values[layer_idx],
            self.sink_pos[layer_idx][:1, 0],
            self.sink_mask[layer_idx],
            self.key_cache[layer_idx],
            self.value_cache[layer_idx],
            self.pos[layer_idx][:1, 0] + pos_shift,
            self.mask[layer_idx],
            self.og_pos[layer_idx],
        )

    def note_tokens_seen(self, layer_idx: int, n_tokens: int):
        """Advance the host mirrors after a kernel advanced the device counter."""
        if layer_idx == 0:
            self._seen_tokens += n_tokens
        self._seen_host[layer_idx] += n_tokens

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               score_states: torch.Tensor = None):
        """Insert ``key_states``/``value_states`` ``[B, H, K, D]`` (any b/h/t strides) in stream order.
        ``score_states`` ``[B, >=H, K]`` are the incoming tokens' scores; ``None`` means all zero
        (the stride rule).  Returns ``get_vals(layer_idx)`` as the reference does."""
        B, H, K, D = key_states.shape
        if (B, H, D) != (self.max_batch_size, self.heads, self.dim) or value_states.shape != key_states.shape:
            raise ValueError(f"key/value shape {tuple(key_states.shape)} does not match the cache "
                             f"({self.max_batch_size}, {self.heads}, K, {self.dim})")
        if K == 0:
            return self.get_vals(layer_idx)
        k, v = self._as_rows(key_states), self._as_rows(value_states)
        if k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
        s_ptr, ss = None, (0, 0, 0)
        if score_states is not None:
            s = score_states
            if s.dim() != 3 or s.size(0) != B or s.size(1) < H or s.size(2) != K:
                raise ValueError(f"score_states shape {tuple(s.shape)}: want [{B}, >={H}, {K}]")
            if s.dtype != self.dtype or s.device != self.device:
                s = s.to(device=self.device, dtype=self.dtype)
            s_ptr, ss = ctypes.c_void_p(s.data_ptr()), s.stride()
        cfg, st = self.ckv_config(layer_idx), self.ckv_state(layer_idx)
        ws_ptr, ws_bytes = None, 0
        if K >= 2 and not self.force_serial_update:
            ws_bytes = self._lib.ckv_update_workspace_bytes(ctypes.byref(cfg), K)
            # the first 256 bytes of the shared workspace stay the attention calls' status word
            self.workspace(ws_bytes + 256)
            ws_ptr = self.workspace_ptr() + 256
        with self.device_guard():
            rc = self._lib.ckv_cascade_update(
                ctypes.byref(cfg), ctypes.byref(st), k.data_ptr(), v.data_ptr(), k.stride(0), k.stride(1),
                k.stride(2), s_ptr, ss[0], ss[1], ss[2], K, ws_ptr, ws_bytes, _lib.current_stream_ptr(self.device))
        _lib.check(rc, "ckv_cascade_update")
        self.note_tokens_seen(layer_idx, K)
        return self.get_vals(layer_idx)

    def _as_rows(self, t: torch.Tensor) -> torch.Tensor:
        """Rows must be contiguous in the last dimension and 16-byte aligned; copy only when they are not."""
        if t.dtype != self.dtype or t.device != self.device:
            t = t.to(device=self.device, dtype=self.dtype)
        esz = t.element_size()
        ok = t.stride(3) == 1 and t.data_ptr() % 16 == 0 and all((t.stride(i) * esz) % 16 == 0 for i in range(3))
        return t if ok else t.contiguous()

    # unsupported HF Cache operations, as in the reference (:1126-1162)
    def to_legacy_cache(self):
        raise NotImplementedError()

    @classmethod
    def from_legacy_cache(cls, past_key_values=None):
        raise NotImplementedError()

    def crop(self, max_length: int):
        raise NotImplementedError()

    def batch_split(self, full_batch_size: int, split_size: int):
        raise NotImplementedError()

    @classmethod
    def from_batch_splits(cls, splits):
        raise NotImplementedError()

    def batch_repeat_interleave(self, repeats: int):
        raise NotImplementedError()

    def batch_select_indices(self, indices: torch.Tensor):
        raise NotImplementedError()

    def reorder_cache(self, beam_idx: torch.LongTensor):
        raise NotImplementedError()

    @property
    def seen_tokens(self):
        raise NotImplementedError()
