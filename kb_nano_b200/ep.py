"""Expert-parallel FP8 MoE layer: host side.

One process per GPU.  `EpMoe` owns the C-side context (symmetric buffers, peer mappings) and calls
`kbn_ep_moe_forward`; torch.distributed is used once, at construction, to exchange the 64-byte CUDA
IPC handles.  The data path never touches NCCL: rows travel by peer stores issued from this
library's kernels.

Expert placement: rank r of R owns the contiguous block of experts [r*E/R, (r+1)*E/R); tokens stay
where they are.  kb-nano shards every expert's intermediate dimension over the ranks instead and
all-reduces the layer output (tasks/baseline/L2/deepseek_moe.py:56,301-302); it has no
expert-parallel layer, so the single-GPU result is what this layer is checked against.
"""
from __future__ import annotations

import ctypes

import torch

from . import _lib
from . import ops as _ops
from .ops import _on, _stream

FP8 = torch.float8_e4m3fn
STATUS_TEXT = {0: "ok", 10: "an expert received more than max_m rows", 11: "expert id out of range",
               20: "timed out waiting for a peer's signal"}


def expert_range(rank: int, world: int, experts_total: int) -> tuple[int, int]:
    if experts_total % world:
        raise ValueError(f"{experts_total} experts do not divide over {world} ranks")
    per = experts_total // world
    return rank * per, (rank + 1) * per


def plan(topk_ids: torch.Tensor, world: int, experts_total: int):
    """(destination rank, local expert index) of every (token, slot) pair -- the placement rule the
    dispatch kernel applies."""
    per = experts_total // world
    ids = topk_ids.long()
    return ids // per, ids % per


class EpStatusError(RuntimeError):
    pass


class EpMoe:
    def __init__(self, rank: int, world: int, experts_total: int, hidden: int, inter: int, max_tokens: int, topk: int,
                 max_m: int = 256, group=None, device: torch.device | None = None, use_ue8m0: bool = True,
                 handles: bytes | None = None):
        """`handles`: the world's 64-byte IPC handles concatenated in rank order, when the caller has exchanged
        them itself (default: all_gather over `group`).  An all-zero handle stands for a rank that never runs
        and is mapped onto this rank's own buffer: waits for it run into their time limit."""
        self.use_ue8m0 = use_ue8m0
        self.rank, self.world = rank, world
        self.experts_total, self.hidden, self.inter = experts_total, hidden, inter
        self.max_tokens, self.topk, self.max_m = max_tokens, topk, max_m
        self.lo, self.hi = expert_range(rank, world, experts_total)
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self._lib = _lib.load()
        self._ctx = ctypes.c_void_p()
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_create(rank, world, experts_total, max_m, hidden, inter, max_tokens, topk,
                                               ctypes.byref(self._ctx)))
            if world > 1 and handles is not None:
                if len(handles) != 64 * world:
                    raise ValueError("handles must hold 64 bytes per rank")
                _lib.check(self._lib.kbn_ep_attach(self._ctx, handles))
            elif world > 1:
                import torch.distributed as dist
                buf = ctypes.create_string_buffer(64)
                _lib.check(self._lib.kbn_ep_ipc_handle(self._ctx, buf))
                handles = [None] * world
                dist.all_gather_object(handles, bytes(buf.raw), group=group)
                blob = b"".join(handles)
                _lib.check(self._lib.kbn_ep_attach(self._ctx, blob))
                dist.barrier(group=group)

    @property
    def symmetric_bytes(self) -> int:
        return int(self._lib.kbn_ep_symmetric_bytes(self._ctx))

    def _check_operands(self, x, w13, w13_s, w2, w2_s):
        e_l = self.hi - self.lo
        if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.hidden or not x.is_contiguous():
            raise ValueError("x must be contiguous bf16 [T, hidden]")
        if tuple(w13.shape) != (e_l, 2 * self.inter, self.hidden) or tuple(w2.shape) != (e_l, self.hidden, self.inter):
            raise ValueError("w13 / w2 must hold this rank's experts: [E/R, 2I, H] and [E/R, H, I]")
        if w13.dtype != FP8 or w2.dtype != FP8 or not w13.is_contiguous() or not w2.is_contiguous():
            raise ValueError("w13 / w2 must be contiguous float8_e4m3fn")
        for s_, n_, k_ in ((w13_s, 2 * self.inter, self.hidden), (w2_s, self.hidden, self.inter)):
            if s_.dtype != torch.float32 or tuple(s_.shape) != (e_l, n_ // 128, k_ // 128) or not s_.is_contiguous():
                raise ValueError("weight scales must be contiguous float32 [E/R, N/128, K/128]")

    def _packed(self, w13_s, w2_s):
        """(p13, p2) packed power-of-two weight scales (checked and packed once per tensor), or (None, None)."""
        if self.use_ue8m0 and self.max_m % 128 == 0:
            p13 = _ops.packed_weight_scales(w13_s, 2 * self.inter, self.hidden)
            p2 = _ops.packed_weight_scales(w2_s, self.hidden, self.inter)
            if p13 is not None and p2 is not None:
                return p13, p2
        return None, None

    def forward_routed(self, x: torch.Tensor, router_logits: torch.Tensor, w13: torch.Tensor, w13_s: torch.Tensor, w2: torch.Tensor,
                       w2_s: torch.Tensor, scoring: str = "softmax", bias: torch.Tensor | None = None, n_group: int = 1,
                       topk_group: int = 1, renormalize: bool = True, renorm_floor: float = 0.0, scale: float = 1.0,
                       round_bf16: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:
        """The layer from the router's logits [T, E] (fp32 or bf16): the dispatch kernel routes on the way (the arguments
        and the arithmetic of ops.moe_route_topk), so the router adds no launch.  `last_routing` returns what it chose."""
        t = x.shape[0]
        self._check_operands(x, w13, w13_s, w2, w2_s)
        if scoring not in ("softmax", "sigmoid"):
            raise ValueError(f"unsupported scoring function {scoring!r}")
        lg = router_logits
        if lg.dim() != 2 or tuple(lg.shape) != (t, self.experts_total) or lg.dtype not in (torch.float32, torch.bfloat16) or lg.stride(1) != 1:
            raise ValueError("router_logits must be fp32 or bf16 [T, experts], contiguous along the experts")
        if lg.device != x.device:
            raise ValueError("router_logits must be on x's device")
        if bias is not None and (bias.dtype != torch.float32 or bias.numel() != self.experts_total or not bias.is_contiguous() or bias.device != x.device):
            raise ValueError("bias must be contiguous float32 [experts] on x's device")
        if out is None:
            out = torch.empty(t, self.hidden, dtype=torch.bfloat16, device=x.device)
        p13, p2 = self._packed(w13_s, w2_s)
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_moe_forward_routed(
                self._ctx, x.data_ptr(), lg.data_ptr(), int(lg.dtype == torch.bfloat16), lg.stride(0) if t > 1 else self.experts_total, t,
                int(scoring == "softmax"), bias.data_ptr() if bias is not None else None, n_group, topk_group, int(renormalize), renorm_floor,
                scale, int(round_bf16), w13.data_ptr(), w13_s.data_ptr(), w2.data_ptr(), w2_s.data_ptr(),
                p13.data_ptr() if p13 is not None else None, p2.data_ptr() if p2 is not None else None, out.data_ptr(), _stream(x)))
        return out

    def last_routing(self, t: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(weights fp32 [t, topk], expert ids int32 [t, topk]) chosen by the last forward_routed call."""
        w = torch.empty(t, self.topk, dtype=torch.float32, device=self.device)
        ids = torch.empty(t, self.topk, dtype=torch.int32, device=self.device)
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_last_routing(self._ctx, w.data_ptr(), ids.data_ptr(), t, torch.cuda.current_stream(self.device).cuda_stream))
        return w, ids

    def forward(self, x: torch.Tensor, topk_ids: torch.Tensor, topk_w: torch.Tensor, w13: torch.Tensor, w13_s: torch.Tensor,
                w2: torch.Tensor, w2_s: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """x bf16 [T,H] (this rank's tokens), topk_ids [T,topk] global expert ids, topk_w [T,topk];
        w13/w2 (+ scales) of this rank's experts only -> bf16 [T,H]."""
        t = x.shape[0]
        self._check_operands(x, w13, w13_s, w2, w2_s)
        ids = topk_ids if topk_ids.dtype == torch.int32 else topk_ids.to(torch.int32)
        ids = ids if ids.is_contiguous() else ids.contiguous()
        w = topk_w if topk_w.dtype == torch.float32 else topk_w.float()
        w = w if w.is_contiguous() else w.contiguous()
        if tuple(ids.shape) != (t, self.topk) or tuple(w.shape) != (t, self.topk):
            raise ValueError("topk_ids / topk_w must be [T, topk]")
        if out is None:
            out = torch.empty(t, self.hidden, dtype=torch.bfloat16, device=x.device)
        # power-of-two weight scales (checked and packed once per tensor) take the UE8M0 GEMM path
        p13, p2 = self._packed(w13_s, w2_s)
        fast = p13 is not None
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_moe_forward(self._ctx, x.data_ptr(), ids.data_ptr(), w.data_ptr(), t, w13.data_ptr(),
                                                    w13_s.data_ptr(), w2.data_ptr(), w2_s.data_ptr(),
                                                    p13.data_ptr() if fast else None, p2.data_ptr() if fast else None,
                                                    out.data_ptr(), _stream(x)))
        return out

    def status(self) -> dict:
        """Synchronises; {code, phase, peer, detail, text}."""
        arr = (ctypes.c_int32 * 4)()
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_status(self._ctx, arr, torch.cuda.current_stream(self.device).cuda_stream))
        code = int(arr[0])
        return {"code": code, "phase": int(arr[1]), "peer": int(arr[2]), "detail": int(arr[3]), "text": STATUS_TEXT.get(code, "unknown")}

    def check(self) -> None:
        s = self.status()
        if s["code"] != 0:
            raise EpStatusError(f"expert-parallel layer on rank {self.rank}: {s}")

    def expert_phase(self, w13: torch.Tensor, w13_s: torch.Tensor, w2: torch.Tensor, w2_s: torch.Tensor,
                     rows_per_expert: torch.Tensor, expected_m: int = 0) -> None:
        """Measurement aid: the two expert GEMMs once more, launched as forward() launches them, on the rows the last
        forward() received, with `rows_per_expert` (int32 [E/R], on the device) as the row counts.  No flags are
        exchanged and the step counter stays, so the call can be bracketed by CUDA events."""
        p13 = _ops.packed_weight_scales(w13_s, 2 * self.inter, self.hidden)
        p2 = _ops.packed_weight_scales(w2_s, self.hidden, self.inter)
        if p13 is None or p2 is None or self.max_m % 128:
            raise ValueError("expert_phase needs power-of-two weight scales and max_m a multiple of 128")
        if rows_per_expert.dtype != torch.int32 or rows_per_expert.numel() != self.hi - self.lo or not rows_per_expert.is_cuda:
            raise ValueError("rows_per_expert must be int32 [E/R] on the device")
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_expert_phase(self._ctx, w13.data_ptr(), p13.data_ptr(), w2.data_ptr(), p2.data_ptr(),
                                                     rows_per_expert.data_ptr(), expected_m, _stream(w13)))

    def clear_status(self) -> None:
        """Sets the status words back to 0 (ordered on the current stream): after an overflow or a time-out has been
        handled, later checks report later steps only."""
        with _on(self.device):
            _lib.check(self._lib.kbn_ep_clear_status(self._ctx, torch.cuda.current_stream(self.device).cuda_stream))

    LAUNCHES_PER_FORWARD = 4   # quantise + dispatch, GEMM1 (+activation), GEMM2 (+combine stores), weighted sum

    def close(self) -> None:
        if self._ctx:
            with _on(self.device):
                self._lib.kbn_ep_destroy(self._ctx)
            self._ctx = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class EpMoeHostPipeline:
    """The layer for callers whose activations and routing live in host memory (a serving loop that samples and
    routes on the CPU, or a test harness): every `submit` copies one step's inputs from pinned host memory to the
    device, runs `EpMoe.forward` and copies the result back to pinned host memory.  The copies run on two streams
    of their own over `depth` rotating device buffers, so the input copy of step i+1 and the result copy of step
    i-1 overlap the layer of step i; only buffer reuse orders them.

    Inputs travel as ONE staged host buffer per step, `blob_bytes` long: bf16 x [T, H], then fp32 topk_w [T, topk],
    then int32 topk_ids [T, topk] (`pack` fills it), with T = the layer's max_tokens.  copy_streams = 1 (the default) puts both
    copies on one stream (a step's result copy is then queued behind the next step's input copy): half the
    cross-stream dependencies per step, which is what an overlapped copy costs (measured: 317 us per step against 333
    with two streams and 293 with device-resident data, for a 7 MB layer step); copy_streams = 2 gives full-duplex PCIe.  `begin` / `join` bracket a
    sequence of submits on the current stream; the whole sequence can be captured in a CUDA graph."""

    def __init__(self, layer: EpMoe, depth: int = 2, copy_streams: int = 1):
        if depth < 1:
            raise ValueError("depth must be at least 1")
        if copy_streams not in (1, 2):
            raise ValueError("copy_streams must be 1 (input and result copies share a stream) or 2")
        self.layer, self.depth = layer, depth
        t, h, k = layer.max_tokens, layer.hidden, layer.topk
        self.nx, self.nw = t * h * 2, t * k * 4
        self.blob_bytes = self.nx + 2 * self.nw
        dev = layer.device
        self._blob = [torch.empty(self.blob_bytes, dtype=torch.uint8, device=dev) for _ in range(depth)]
        self._out = [torch.empty(t, h, dtype=torch.bfloat16, device=dev) for _ in range(depth)]
        self._views = [(b[:self.nx].view(torch.bfloat16).view(t, h), b[self.nx:self.nx + self.nw].view(torch.float32).view(t, k),
                        b[self.nx + self.nw:].view(torch.int32).view(t, k)) for b in self._blob]
        self._s_in = torch.cuda.Stream(dev)
        self._s_out = torch.cuda.Stream(dev) if copy_streams == 2 else self._s_in
        self._ev_fw = [None] * depth      # forward that last read _blob[b] and wrote _out[b]
        self._ev_out = [None] * depth     # result copy that last read _out[b]
        self._pending = None              # (host_out, buffer) of a step whose result copy is not queued yet
        self._n = 0

    def new_host_buffers(self) -> tuple[torch.Tensor, torch.Tensor]:
        t, h = self.layer.max_tokens, self.layer.hidden
        return torch.empty(self.blob_bytes, dtype=torch.uint8).pin_memory(), torch.empty(t, h, dtype=torch.bfloat16).pin_memory()

    def pack(self, blob: torch.Tensor, x: torch.Tensor, topk_w: torch.Tensor, topk_ids: torch.Tensor) -> None:
        t, h, k = self.layer.max_tokens, self.layer.hidden, self.layer.topk
        blob[:self.nx].view(torch.bfloat16).view(t, h).copy_(x)
        blob[self.nx:self.nx + self.nw].view(torch.float32).view(t, k).copy_(topk_w)
        blob[self.nx + self.nw:].view(torch.int32).view(t, k).copy_(topk_ids)

    def begin(self) -> None:
        """The copy streams start after everything already queued on the current stream."""
        cur = torch.cuda.current_stream(self.layer.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        self._s_in.wait_event(ev)
        self._s_out.wait_event(ev)
        self._ev_fw = [None] * self.depth
        self._ev_out = [None] * self.depth
        self._pending = None
        self._n = 0

    def _flush_result(self) -> None:
        if self._pending is None:
            return
        host_out, b = self._pending
        self._pending = None
        self._s_out.wait_event(self._ev_fw[b])
        with torch.cuda.stream(self._s_out):
            host_out.copy_(self._out[b], non_blocking=True)
            self._ev_out[b] = torch.cuda.Event()
            self._ev_out[b].record(self._s_out)

    def submit(self, host_blob: torch.Tensor, host_out: torch.Tensor, w13, w13_s, w2, w2_s) -> None:
        if not (host_blob.is_pinned() and host_out.is_pinned()):
            raise ValueError("host buffers must be pinned")
        if host_blob.numel() != self.blob_bytes or host_blob.dtype != torch.uint8:
            raise ValueError(f"host_blob must be uint8 [{self.blob_bytes}]")
        b = self._n % self.depth
        self._n += 1
        cur = torch.cuda.current_stream(self.layer.device)
        if self._ev_fw[b] is not None:
            self._s_in.wait_event(self._ev_fw[b])
        with torch.cuda.stream(self._s_in):
            self._blob[b].copy_(host_blob, non_blocking=True)
            ev_in = torch.cuda.Event()
            ev_in.record(self._s_in)
        # one copy stream: the previous step's result copy (which waits for that step's layer) is queued behind this
        # step's input copy, so that the input copy is not held up by it
        self._flush_result()
        cur.wait_event(ev_in)
        if self._ev_out[b] is not None:
            cur.wait_event(self._ev_out[b])
        x, tw, ti = self._views[b]
        self.layer.forward(x, ti, tw, w13, w13_s, w2, w2_s, out=self._out[b])
        self._ev_fw[b] = torch.cuda.Event()
        self._ev_fw[b].record(cur)
        self._pending = (host_out, b)
        if self._s_out is not self._s_in:
            self._flush_result()

    def join(self) -> None:
        """The current stream waits for every copy submitted since `begin`."""
        self._flush_result()
        cur = torch.cuda.current_stream(self.layer.device)
        for ev in self._ev_out:
            if ev is not None:
                cur.wait_event(ev)
        ev = torch.cuda.Event()
        ev.record(self._s_in)
        cur.wait_event(ev)
