"""The `cuda` module's runtime function: executes a quantized program on one B200.

Mirrors what a ``runtime_function`` subclass does in the reference's native runtime
(``initialize_core`` = upload weights and plan buffers once; ``invoke_core`` = run the kernels
for one call, src/Native/include/nncase/runtime/runtime_function.h:59-63): tensors cross the
boundary as f32 NCHW host or device arrays, stay u8 NHWC inside, and nothing is allocated or
uploaded per call. The per-op host loop of the reference's StackVM
(runtime_function.run.cpp:34-63) is replaced by a pre-planned launch list that can be captured
into a CUDA graph.
"""
import numpy as np
import torch

from . import lib as L
from .kernels import Context, NncbError, QuantParam

INF = float("inf")


class CudaFunction:
    def __init__(self, program, batch, ctx=None, device=0, force_path=L.PATH_AUTO):
        self.ctx = ctx or Context(device)
        self.program = program
        self.batch = batch
        dev = self.ctx.device
        self.buffers = {}
        for name, t in program["tensors"].items():
            h, w, c = t["shape"]
            dt = torch.uint8 if t["dtype"] == "u8" else torch.float32
            self.buffers[name] = torch.empty((batch, h, w, c), dtype=dt, device=dev)
        self.steps = []
        self.plans = []
        for op in program["ops"]:
            self.steps.append(self._plan(op, force_path))
        in_t = program["tensors"][program["input"]]
        self.in_qp = in_t["qp"]
        self._graph = None
        self.pipeline_graphs = True   # submit_host replays one captured graph per staging buffer
        self._static_in = None
        self.launches_per_call = None

    # ---- planning --------------------------------------------------------------------------
    def _plan(self, op, force_path):
        ctx, buf, T = self.ctx, self.buffers, self.program["tensors"]
        kind = op["op"]
        if kind == "quantize_input":
            return ("quantize_input", op)
        if kind == "conv":
            tin = T[op["in"]]
            h, w, c = tin["shape"]
            residual = y2 = None
            out_qp = op["conv_qp"]
            if op.get("res"):
                residual = (T[op["res"]]["qp"], T[op["out"]]["qp"])
            if op.get("y2"):
                y2 = (T[op["y2"]]["qp"], 0.0, INF)
            plan = ctx.conv2d_plan((self.batch, h, w, c), op["w"], op["w_zp"], op["mult"], op["bias"],
                                   tin["qp"].zero_point, out_qp, stride=op["stride"], padding=op["pad"],
                                   dilation=op["dil"], groups=op["groups"], fused_clamp=op["clamp"], residual=residual,
                                   y2=y2, f32_out=bool(op.get("f32_out")), force_path=force_path, lut=op.get("lut"))
            self.plans.append(plan)
            return ("conv", op, plan)
        if kind == "concat":
            # one requantising table per input: into the concat's quant param
            tables, off = [], 0
            oq = T[op["out"]]["qp"]
            for name in op["ins"]:
                iq = T[name]["qp"]
                t = np.empty(256, np.uint8)
                L.check(ctx._lib.nncb_make_requant_table(iq.scale, iq.zero_point, oq.scale, oq.zero_point,
                                                         -INF, INF, t.ctypes.data))
                identity = (iq.scale, iq.zero_point) == (oq.scale, oq.zero_point)
                tables.append((name, off, T[name]["shape"][2], None if identity else t))
                off += T[name]["shape"][2]
            return ("concat", op, tables)
        if kind in ("maxpool", "requant", "gap", "add", "slice", "upsample"):
            return (kind, op)
        raise NncbError(-38, f"unsupported program op {kind}")

    @property
    def conv_paths(self):
        """{layer name: 1 (CUDA cores) | 2 (tcgen05)}"""
        return {s[1]["name"]: s[2].path for s in self.steps if s[0] == "conv"}

    # ---- execution -------------------------------------------------------------------------
    def _run(self, x_dev):
        """Enqueue all kernels of one call; x_dev: f32 NCHW device tensor of the planned batch."""
        ctx, buf, T = self.ctx, self.buffers, self.program["tensors"]
        lib, h_ = ctx._lib, ctx._h
        for st in self.steps:
            kind, op = st[0], st[1]
            if kind == "quantize_input":
                n, c, hh, ww = x_dev.shape
                qp = T[op["out"]]["qp"]
                if op.get("s2d") and any(op.get("pad", ())):
                    if op.get("nhwc"):
                        n, hh, ww, c = x_dev.shape
                    else:
                        n, c, hh, ww = x_dev.shape
                    pt, pb, pl, pr = op["pad"]
                    L.check(lib.nncb_quantize_to_s2d_padded_u8(h_, x_dev.data_ptr(), int(bool(op.get("nhwc"))),
                                                               buf[op["out"]].data_ptr(), n, c, hh, ww, op["c_pad"], pt, pb,
                                                               pl, pr, qp.scale, qp.zero_point))
                elif op.get("nhwc"):
                    n, hh, ww, c = x_dev.shape
                    if op.get("s2d"):
                        L.check(lib.nncb_quantize_nhwc_to_s2d_u8(h_, x_dev.data_ptr(), buf[op["out"]].data_ptr(), n, hh, ww,
                                                                 c, op["c_pad"], qp.scale, qp.zero_point))
                    elif op["c_pad"] == c:
                        L.check(lib.nncb_quantize(h_, x_dev.data_ptr(), buf[op["out"]].data_ptr(), x_dev.numel(),
                                                  qp.scale, qp.zero_point, L.U8))
                    else:
                        raise NncbError(-38, "NHWC input with channel padding is only built for stride-2 stems")
                else:
                    fn_q = lib.nncb_quantize_nchw_to_s2d_u8 if op.get("s2d") else lib.nncb_quantize_nchw_to_nhwc_u8
                    L.check(fn_q(h_, x_dev.data_ptr(), buf[op["out"]].data_ptr(), n, c, hh, ww, op["c_pad"], qp.scale,
                                 qp.zero_point))
            elif kind == "conv":
                plan = st[2]
                res = buf[op["res"]] if op.get("res") else None
                y2 = buf[op["y2"]] if op.get("y2") else None
                L.check(lib.nncb_qconv2d_run(h_, plan._h, buf[op["in"]].data_ptr(),
                                             res.data_ptr() if res is not None else None, buf[op["out"]].data_ptr(),
                                             y2.data_ptr() if y2 is not None else None))
            elif kind == "maxpool":
                hh, ww, c = T[op["in"]]["shape"]
                L.check(lib.nncb_maxpool_u8(h_, buf[op["in"]].data_ptr(), buf[op["out"]].data_ptr(), self.batch, hh, ww, c,
                                            op["k"][0], op["k"][1], op["stride"][0], op["stride"][1], *op["pad"],
                                            T[op["in"]]["qp"].zero_point))
            elif kind == "requant":
                qi, qo = T[op["in"]]["qp"], T[op["out"]]["qp"]
                L.check(lib.nncb_requant_u8(h_, buf[op["in"]].data_ptr(), buf[op["out"]].data_ptr(),
                                            buf[op["in"]].numel(), qi.scale, qi.zero_point, qo.scale, qo.zero_point,
                                            op["clamp"][0], op["clamp"][1]))
            elif kind == "add":
                qa, qb, qo = T[op["a"]]["qp"], T[op["b"]]["qp"], T[op["out"]]["qp"]
                L.check(lib.nncb_qadd_u8(h_, buf[op["a"]].data_ptr(), buf[op["b"]].data_ptr(), buf[op["out"]].data_ptr(),
                                         buf[op["out"]].numel(), qa.scale, qa.zero_point, qb.scale, qb.zero_point,
                                         qo.scale, qo.zero_point))
            elif kind == "slice":
                hh, ww, c = T[op["in"]]["shape"]
                L.check(lib.nncb_copy_channels_u8(h_, buf[op["in"]].data_ptr(), c, op["begin"], buf[op["out"]].data_ptr(),
                                                  op["end"] - op["begin"], 0, op["end"] - op["begin"],
                                                  self.batch * hh * ww, None))
            elif kind == "concat":
                hh, ww, ctot = T[op["out"]]["shape"]
                for name, off, ci, table in st[2]:
                    L.check(lib.nncb_copy_channels_u8(h_, buf[name].data_ptr(), ci, 0, buf[op["out"]].data_ptr(), ctot, off,
                                                      ci, self.batch * hh * ww,
                                                      table.ctypes.data if table is not None else None))
            elif kind == "upsample":
                hh, ww, c = T[op["in"]]["shape"]
                L.check(lib.nncb_resize_nearest_u8(h_, buf[op["in"]].data_ptr(), buf[op["out"]].data_ptr(), self.batch, hh,
                                                   ww, c, op["factor"], op["factor"]))
            elif kind == "gap":
                hh, ww, c = T[op["in"]]["shape"]
                qi, qo = T[op["in"]]["qp"], T[op["out"]]["qp"]
                L.check(lib.nncb_global_avgpool_u8(h_, buf[op["in"]].data_ptr(), buf[op["out"]].data_ptr(), self.batch,
                                                   hh, ww, c, qi.scale, qi.zero_point, qo.scale, qo.zero_point))
        return buf[self.program["output"]]

    def invoke(self, x_dev):
        """Device in (f32 NCHW [batch,c,h,w]), device out (the program's output buffer)."""
        if x_dev.shape[0] != self.batch or x_dev.dtype != torch.float32 or not x_dev.is_contiguous():
            raise NncbError(-22, "invoke: input must be a contiguous f32 tensor of the planned batch")
        self.ctx.use_current_stream()
        before = self.ctx.launches
        out = self._run(x_dev)
        self.launches_per_call = self.ctx.launches - before
        return out

    def capture(self, x_dev):
        """Capture one call into a CUDA graph reading from a static copy of x_dev's storage."""
        self._static_in = x_dev.clone()
        self.invoke(self._static_in)  # warm-up outside capture (tensor maps, lazy init)
        torch.cuda.synchronize(self.ctx.device)
        g = torch.cuda.CUDAGraph()
        # thread-local capture: another thread of the process (a collective library's watchdog) may call the runtime
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            self.ctx.use_current_stream()
            self._run(self._static_in)
        self.ctx.use_current_stream()
        self._graph = g
        return g

    def replay(self, x_dev=None):
        if x_dev is not None:
            self._static_in.copy_(x_dev, non_blocking=True)
        self._graph.replay()
        return self.buffers[self.program["output"]]

    def invoke_host(self, x_host, out_host=None, pinned_in=None):
        """Host in, host out (numpy or pinned torch tensors): H2D copy, kernels, D2H copy, sync."""
        x = torch.as_tensor(x_host)
        xd = x.to(self.ctx.device, non_blocking=True)
        out = self.replay(xd) if self._graph is not None else self.invoke(xd)
        if out_host is None:
            res = out.to("cpu")
        else:
            out_host.copy_(out, non_blocking=True)
            res = out_host
        torch.cuda.current_stream(self.ctx.device).synchronize()
        return res

    # ---- pipelined host-buffer calls -------------------------------------------------------
    # A caller that feeds batch after batch from host memory does not want invoke_host's
    # copy-in / run / copy-out / wait per batch: submit_host() queues one batch and returns at once.
    # Two device staging buffers and two streams overlap the host-to-device copy of batch i+1 with
    # the kernels of batch i; results land in the caller's host buffer, valid after drain() (or after
    # the event submit_host returns has completed).
    def _pipeline(self):
        if getattr(self, "_pipe", None) is None:
            dev = self.ctx.device
            in_t = self.program["tensors"][self.program["input"]]
            self._pipe = dict(copy=torch.cuda.Stream(dev), comp=torch.cuda.Stream(dev), xd=[None, None],
                              copied=[torch.cuda.Event(), torch.cuda.Event()],
                              done=[torch.cuda.Event(), torch.cuda.Event()], n=0, graphs=[None, None], uses=[0, 0])
        return self._pipe

    def submit_host(self, x_host, out_host):
        """Queue one batch: x_host (f32, pinned torch tensor of the planned input shape) -> out_host (pinned
        torch tensor shaped like the program's output). Returns the event that marks out_host valid."""
        if not (x_host.is_pinned() and out_host.is_pinned()):
            raise NncbError(-22, "submit_host: both host tensors must be pinned (torch.Tensor.pin_memory)")
        if x_host.shape[0] != self.batch or x_host.dtype != torch.float32 or not x_host.is_contiguous():
            raise NncbError(-22, "submit_host: input must be a contiguous f32 tensor of the planned batch")
        p = self._pipeline()
        b = p["n"] & 1
        if p["xd"][b] is None or p["xd"][b].shape != x_host.shape:
            p["xd"][b] = torch.empty(x_host.shape, dtype=torch.float32, device=self.ctx.device)
            p["graphs"][b], p["uses"][b] = None, 0
        with torch.cuda.stream(p["copy"]):
            if p["n"] >= 2:
                p["copy"].wait_event(p["done"][b])     # the kernels that read this staging buffer two batches ago
            p["xd"][b].copy_(x_host, non_blocking=True)
            p["copied"][b].record()
        with torch.cuda.stream(p["comp"]):
            p["comp"].wait_event(p["copied"][b])
            self.ctx.use_current_stream()
            if p["graphs"][b] is not None:
                p["graphs"][b].replay()              # the kernels of one call, reading this staging buffer
                out = self.buffers[self.program["output"]]
            else:
                before = self.ctx.launches
                out = self._run(p["xd"][b])
                self.launches_per_call = self.ctx.launches - before
            out_host.copy_(out, non_blocking=True)
            p["done"][b].record()
        p["uses"][b] += 1
        if p["graphs"][b] is None and p["uses"][b] == 1 and self.pipeline_graphs:
            # the first batch through a staging buffer has run eagerly (plans and tensor maps are warm): capture the
            # launch list once per buffer; later batches replay it (one graph launch instead of one call per operator)
            p["comp"].synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=p["comp"], capture_error_mode="thread_local"):
                self.ctx.use_current_stream()
                self._run(p["xd"][b])
            p["graphs"][b] = g
        p["n"] += 1
        return p["done"][b]

    def drain(self):
        """Wait for every batch queued with submit_host; re-binds the context to the caller's stream."""
        p = self._pipeline()
        p["comp"].synchronize()
        p["copy"].synchronize()
        self.ctx.use_current_stream()

    def tensor(self, name):
        return self.buffers[name]

    def outputs(self):
        """The program's output tensors, in order (u8 NHWC, or f32 for a MatMul classifier)."""
        return [self.buffers[n] for n in self.program.get("outputs", [self.program["output"]])]

    def close(self):
        if getattr(self, "_pipe", None) is not None:
            self.drain()
            self._pipe["graphs"] = [None, None]
        for p in self.plans:
            p.close()
        self.plans = []
