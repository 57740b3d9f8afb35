"""Weight-gradient GEMM on the tcgen05 tensor cores (csrc/kernels/wgrad_gemm.cu).

    dW = wgrad_gemm(dY, X)          # dY [tokens, out], X [tokens, in], bf16 -> dW [out, in] fp32

``FusedWgrad`` additionally sums dW over all workers inside the same kernel: the output
lives in the symmetric heap, every finished tile is reduced through the NVSwitch while
later tiles are still being computed.
"""
import ctypes
import os

import torch

from .._native import library_path, NativeError

_LIB = None
_TWO_CTA_DEFAULT = True   # measured: 53 vs 58 us on 8192x4096x1024, 815 vs 923 us on 8192^3


class _FusedArgs(ctypes.Structure):
    _fields_ = [("rank", ctypes.c_int), ("nranks", ctypes.c_int),
                ("flags_peer", ctypes.c_void_p * 8), ("out_mc", ctypes.c_void_p),
                ("epoch", ctypes.c_ulonglong), ("timeout_ns", ctypes.c_ulonglong),
                ("scale", ctypes.c_float), ("work_counter", ctypes.c_void_p),
                ("mode", ctypes.c_int), ("gather_local", ctypes.c_void_p), ("gather_mc", ctypes.c_void_p),
                ("gather_counter", ctypes.c_void_p)]


def _lib():
    global _LIB
    if _LIB is None:
        path = library_path("libswitchml_gemm.so")
        if not os.path.exists(path):
            raise ImportError("libswitchml_gemm.so is not built (run build.py)")
        l = ctypes.CDLL(path)
        l.switchml_wgrad_gemm.restype = ctypes.c_int
        l.switchml_wgrad_gemm.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                          ctypes.c_int, ctypes.c_int, ctypes.POINTER(_FusedArgs),
                                          ctypes.c_void_p, ctypes.c_void_p]
        l.switchml_wgrad_gemm_2cta.restype = ctypes.c_int
        l.switchml_wgrad_gemm_2cta.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int,
                                               ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        l.switchml_wgrad_flag_words.restype = ctypes.c_int
        l.switchml_wgrad_flag_words.argtypes = [ctypes.c_int, ctypes.c_int]
        _LIB = l
    return _LIB


_ERRORS = {-1: "bad argument", -2: "M and N must be multiples of 8 and all tensors 16-byte aligned",
           -3: "cannot build the TMA tensor maps", -4: "kernel launch failed"}


def wgrad_gemm(dy, x, out=None, error_flag=None, two_cta=None):
    """dW[out_features, in_features] (fp32) = dY^T @ X for bf16 dY [K, M] and X [K, N].

    `two_cta`: use the kernel in which two CTAs share a 256x256 tile (tcgen05 cta_group::2);
    default: whenever the reduction dimension is at least 256, where shared-memory bandwidth
    bounds the one-CTA kernel."""
    assert dy.is_cuda and x.is_cuda and dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
    assert dy.dim() == 2 and x.dim() == 2 and dy.shape[0] == x.shape[0]
    dy = dy.contiguous()
    x = x.contiguous()
    K, M = dy.shape
    N = x.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=dy.device)
    assert out.is_contiguous() and out.dtype == torch.float32 and out.numel() == M * N
    stream = torch.cuda.current_stream(dy.device).cuda_stream
    err_ptr = error_flag.data_ptr() if error_flag is not None else None
    if two_cta is None:
        two_cta = _TWO_CTA_DEFAULT and K >= 256   # tiny K is output-bound: the one-CTA kernel wins there
    if two_cta:
        rc = _lib().switchml_wgrad_gemm_2cta(dy.data_ptr(), x.data_ptr(), out.data_ptr(), M, N, K, err_ptr,
                                             ctypes.c_void_p(stream))
    else:
        rc = _lib().switchml_wgrad_gemm(dy.data_ptr(), x.data_ptr(), out.data_ptr(), M, N, K, None, err_ptr,
                                        ctypes.c_void_p(stream))
    if rc != 0:
        raise NativeError("wgrad_gemm: " + _ERRORS.get(rc, str(rc)))
    return out.view(M, N)


def flag_words(M, N):
    return _lib().switchml_wgrad_flag_words(M, N)


class FusedWgrad:
    """Weight-gradient GEMM whose result is summed over all workers inside the kernel.

    One instance per weight matrix [M, N]. The gradient buffer and the tile flags live in
    the context's symmetric heap (every rank must create its instances in the same order).
    ``run(dy, x)`` leaves the reduced (scaled) gradient in ``self.grad`` on every rank; the
    kernel is enqueued on the current stream and needs no separate allreduce.
    """

    def __init__(self, ctx, M, N, scale=1.0, timeout_ms=20000.0, policy="auto"):
        self.ctx, self.M, self.N, self.scale = ctx, M, N, scale
        self.grad = ctx.symmetric_empty(M * N, torch.float32).view(M, N)
        words = flag_words(M, N)
        self.flags = ctx.symmetric_empty(words * 2, torch.int32)   # 64-bit words
        self.flags.zero_()
        self.error = torch.zeros(1, dtype=torch.int32, device=self.grad.device)
        local, peers, mc, _ = ctx.symmetric_info()
        self.nranks = sum(1 for p in peers if p)
        self.rank = peers.index(local)
        self.args = _FusedArgs()
        self.args.rank, self.args.nranks = self.rank, self.nranks
        flag_off = self.flags.data_ptr() - local
        for r in range(self.nranks):
            self.args.flags_peer[r] = peers[r] + flag_off
        self.args.out_mc = (mc + (self.grad.data_ptr() - local)) if mc else None
        self.args.epoch = 0
        self.args.timeout_ns = int(timeout_ms * 1e6)
        self.args.scale = scale
        self.counter = torch.zeros(1, dtype=torch.int32, device=self.grad.device)
        self.args.work_counter = self.counter.data_ptr()
        self.fused = self.nranks > 1 and bool(mc)
        self._symm = (local, mc)
        self.gather_buf = None     # [nranks * K * (M + N)] bf16 in the symmetric heap, made on first use
        self.gather_k = 0
        self.gather_counter = torch.zeros(1, dtype=torch.int32, device=self.grad.device)
        self.args.gather_counter = self.gather_counter.data_ptr()
        # "gather": the ranks exchange their (small) operands, every rank computes the tiles it
        # owns over all of them and broadcasts them: the gradient crosses the link once;
        # "fused": every rank multiplies its own operands and finished tiles are reduced through
        # the switch inside the GEMM kernel; "split": GEMM, then the in-place reduction as a
        # second kernel; "auto": gather when the operands of all ranks are less than a quarter of
        # the gradient (VGG's fully connected layers, K = batch), else split, which measured
        # faster than the fused reduction for long K.
        self.policy = policy
        torch.cuda.synchronize()

    def run(self, dy, x, side_stream=None):
        """Compute (and reduce) the gradient. With `side_stream` the kernel runs there,
        ordered after the current stream; call ``wait_pending()`` before using the result.
        Nothing later in backward needs dW, so this keeps the reduction off the critical path."""
        assert dy.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
        dy, x = dy.contiguous(), x.contiguous()
        if side_stream is not None:
            side_stream.wait_stream(torch.cuda.current_stream(dy.device))
            dy.record_stream(side_stream)
            x.record_stream(side_stream)
            with torch.cuda.stream(side_stream):
                out = self.run(dy, x)
                ev = torch.cuda.Event()
                ev.record(side_stream)
            _PENDING.append(ev)
            return out
        K = dy.shape[0]
        operand_bytes = self.nranks * K * (self.M + self.N) * 2
        gather = self.fused and (self.policy == "gather" or
                                 (self.policy == "auto" and 4 * operand_bytes <= self.M * self.N * 4))
        in_kernel = gather or (self.fused and self.policy == "fused")
        if gather and (self.gather_buf is None or self.gather_k != K):
            # every rank gets here with the same shapes in the same order, so the symmetric
            # allocations stay in step
            try:
                self.gather_buf = self.ctx.symmetric_empty(self.nranks * K * (self.M + self.N), torch.bfloat16)
            except MemoryError:
                # the heap is used up (it is never freed piecemeal); every rank sees the same heap,
                # so every rank falls back to the two-kernel path for this shape
                self.gather_buf, gather, in_kernel = None, False, self.fused and self.policy == "fused"
            else:
                self.gather_k = K
                local, mc = self._symm
                self.args.gather_local = self.gather_buf.data_ptr()
                self.args.gather_mc = mc + (self.gather_buf.data_ptr() - local)
        self.args.mode = 1 if gather else 0
        if in_kernel:
            self.args.epoch += 1
            self.counter.zero_()  # work queue of the in-kernel reduction starts at zero
            stream = torch.cuda.current_stream(dy.device).cuda_stream
            rc = _lib().switchml_wgrad_gemm(dy.data_ptr(), x.data_ptr(), self.grad.data_ptr(), self.M, self.N, K,
                                            ctypes.byref(self.args), self.error.data_ptr(), ctypes.c_void_p(stream))
            if rc != 0:
                raise NativeError("wgrad_gemm: " + _ERRORS.get(rc, str(rc)))
        else:
            wgrad_gemm(dy, x, out=self.grad, error_flag=self.error)
        if not in_kernel and self.nranks > 1:
            # No multicast mapping: reduce the finished gradient with the zero-copy kernel.
            job = self.ctx.all_reduce_async(self.grad.view(-1))
            job.stream_wait()
            job.release()
            if self.scale != 1.0:
                self.grad.mul_(self.scale)
        return self.grad


_PENDING = []
_SIDE_STREAMS = {}


def wait_pending(stream=None):
    """Order `stream` (default: current) after every weight-gradient kernel that was sent to
    a side stream since the last call."""
    if not _PENDING:
        return
    s = stream or torch.cuda.current_stream()
    while _PENDING:
        s.wait_event(_PENDING.pop())


def _side_stream(device):
    if device not in _SIDE_STREAMS:
        _SIDE_STREAMS[device] = torch.cuda.Stream(device=device, priority=-1)
    return _SIDE_STREAMS[device]


class _FusedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        ctx.layer = layer
        ctx.save_for_backward(x, weight)
        return torch.nn.functional.linear(x, weight, bias)

    @staticmethod
    def backward(ctx, dy):
        x, weight = ctx.saved_tensors
        layer = ctx.layer
        x2 = x.reshape(-1, x.shape[-1])
        dy2 = dy.reshape(-1, dy.shape[-1])
        dx = (dy2 @ weight.to(dy2.dtype)).reshape(x.shape) if ctx.needs_input_grad[0] else None
        # dW on the tcgen05 tensor cores, summed over the workers in the same kernel,
        # written straight into the parameter's gradient.
        layer.wgrad.run(dy2.to(torch.bfloat16), x2.to(torch.bfloat16),
                        side_stream=_side_stream(dy2.device) if layer.overlap else None)
        dbias = dy2.sum(0).to(layer.bias.dtype) if layer.bias is not None else None
        return dx, None, dbias, None


class FusedWgradLinear(torch.nn.Linear):
    """``nn.Linear`` whose weight gradient is computed by ``FusedWgrad`` (fp32 weights,
    bf16 activations). Call ``attach(ctx)`` once after the context has started; the weight's
    ``.grad`` then aliases the symmetric gradient buffer and arrives already reduced."""

    wgrad = None
    overlap = True  # run the weight-gradient kernel on a side stream

    def attach(self, ctx, scale=1.0):
        self.wgrad = FusedWgrad(ctx, self.out_features, self.in_features, scale)
        self.weight.grad = self.wgrad.grad
        self.weight._sml_reduced_in_backward = True
        return self

    def forward(self, x):
        if self.wgrad is None or not torch.is_grad_enabled():
            return super().forward(x)
        w = self.weight
        if torch.is_autocast_enabled():
            dt = torch.get_autocast_dtype("cuda")
            return _FusedLinearFn.apply(x.to(dt), w.to(dt), self.bias.to(dt) if self.bias is not None else None, self)
        return _FusedLinearFn.apply(x, w, self.bias, self)
