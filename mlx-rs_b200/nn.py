"""Module layer: SwitchGlu and MoeBlock with the forward signatures the reference's modules use.

`forward` mirrors `Module::forward` (mlx-rs/src/module/module.rs:27-44; template
mlx-lm/src/models/qwen3.rs:204-255): MoeBlock.forward(x [B,L,H]) -> [B,L,H],
SwitchGlu.forward(x [..,H], indices [..,k]) -> [..,k,H].  Parameters keep the QuantizedLinear
field names weight / scales / biases, group_size, bits (mlx-rs/src/nn/quantized.rs:307-335)
stacked over experts.
"""
import ctypes as C
from dataclasses import dataclass

import torch

from . import _lib as L
from . import ops

ROUTER_SOFTMAX_TOPK = 0
ROUTER_TOPK_SOFTMAX = 1


@dataclass
class QuantizedSwitchLinear:
    """Stacked quantized projection: weight [E,out,in*bits/32] int32, scales/biases [E,out,in/gs] bf16."""
    weight: torch.Tensor
    scales: torch.Tensor
    biases: torch.Tensor
    group_size: int = ops.DEFAULT_GROUP_SIZE
    bits: int = ops.DEFAULT_BITS

    @classmethod
    def from_weight(cls, w, group_size=ops.DEFAULT_GROUP_SIZE, bits=ops.DEFAULT_BITS, ctx=None):
        """Quantizable::try_into_quantized (mlx-rs/src/quantization.rs:6-25) for a stacked [E,out,in] weight."""
        return cls(*ops.quantize(w, group_size, bits, ctx=ctx), group_size=group_size, bits=bits)

    def forward(self, x, indices, sorted_indices=False, ctx=None):
        """x [n,1,in] (or [n,in]), indices [n] -> [n,1,out] via gather_qmm(transpose=true)."""
        x3 = x if x.dim() == 3 else x.unsqueeze(-2)
        y = ops.gather_qmm(x3, self.weight, self.scales, self.biases, None, indices, True, self.group_size, self.bits,
                           sorted_indices, ctx=ctx)
        return y if x.dim() == 3 else y.squeeze(-2)

    def c_struct(self):
        return L.QLinear(self.weight.data_ptr(), self.scales.data_ptr(), self.biases.data_ptr())


class SwitchGlu:
    def __init__(self, gate_proj, up_proj, down_proj, ctx=None):
        self.gate_proj, self.up_proj, self.down_proj = gate_proj, up_proj, down_proj
        self.ctx = ctx
        E, I, _ = gate_proj.weight.shape
        H = down_proj.weight.shape[1]
        self.hidden, self.inter, self.n_experts = H, I, E

    def _cfg(self, top_k, router_mode=0, norm_topk_prob=True):
        return L.MoeConfig(self.hidden, self.inter, self.n_experts, top_k, self.gate_proj.bits, self.gate_proj.group_size,
                           router_mode, int(norm_topk_prob))

    def _params(self, router_weight=None, logit_bias=None):
        return L.MoeParams(router_weight.data_ptr() if router_weight is not None else None,
                           logit_bias.data_ptr() if logit_bias is not None else None, self.gate_proj.c_struct(),
                           self.up_proj.c_struct(), self.down_proj.c_struct())

    def forward(self, x, indices):
        ops._cuda(x, indices)
        ops._req(x.dtype == torch.bfloat16 and indices.dtype == torch.int32, "SwitchGlu: bf16 x, int32 indices")
        k = indices.shape[-1]
        T = indices.numel() // k
        out = torch.empty(tuple(indices.shape) + (self.hidden,), dtype=x.dtype, device=x.device)
        cfg, params = self._cfg(k), self._params()
        L.check(L.lib().b200_switch_glu_forward(ops._ctx(self.ctx), C.byref(cfg), C.byref(params), L.ptr(x),
                                                L.ptr(indices), T, L.ptr(out), L.stream_ptr()))
        return out


    def forward_sorted(self, rows, counts, n=None, out=None):
        """SwitchGLU over rows already grouped by expert (counts[e] consecutive rows each): the
        sorted-input case, without the sort.  `out` may be a preallocated [n, hidden] bf16 buffer."""
        ops._cuda(rows, counts)
        ops._req(rows.dtype == torch.bfloat16 and counts.dtype == torch.int32, "forward_sorted: bf16 rows, int32 counts")
        n = rows.shape[0] if n is None else n
        if out is None:
            out = torch.empty((n, self.hidden), dtype=rows.dtype, device=rows.device)
        cfg, params = self._cfg(1), self._params()
        L.check(L.lib().b200_switch_glu_sorted(ops._ctx(self.ctx), C.byref(cfg), C.byref(params), L.ptr(rows),
                                               L.ptr(counts), n, L.ptr(out), L.stream_ptr()))
        return out


    def forward_sorted_scatter(self, rows, counts, n, out_row_addr):
        """forward_sorted whose output rows go to the per-row addresses `out_row_addr` (int64 [n], bf16 rows of
        `hidden` elements each; the addresses may be in peer GPUs' memory)."""
        ops._cuda(rows, counts, out_row_addr)
        ops._req(rows.dtype == torch.bfloat16 and counts.dtype == torch.int32 and out_row_addr.dtype == torch.int64,
                 "forward_sorted_scatter: bf16 rows, int32 counts, int64 addresses")
        cfg, params = self._cfg(1), self._params()
        L.check(L.lib().b200_switch_glu_sorted_scatter(ops._ctx(self.ctx), C.byref(cfg), C.byref(params), L.ptr(rows),
                                                       L.ptr(counts), n, L.ptr(out_row_addr), L.stream_ptr()))


class MoeBlock:
    """gate (router Linear, weight [E,H] bf16) + switch_mlp (SwitchGlu)."""

    def __init__(self, gate_weight, switch_mlp, top_k, norm_topk_prob=True, router_mode=ROUTER_SOFTMAX_TOPK,
                 router_logit_bias=None, ctx=None):
        self.gate_weight, self.switch_mlp = gate_weight, switch_mlp
        self.top_k, self.norm_topk_prob, self.router_mode = top_k, norm_topk_prob, router_mode
        self.router_logit_bias = router_logit_bias
        self.ctx = ctx
        self._cfg = switch_mlp._cfg(top_k, router_mode, norm_topk_prob)
        self._params = switch_mlp._params(gate_weight, router_logit_bias)

    @property
    def config(self):
        return self._cfg

    def forward(self, x, return_aux=False, out=None):
        ops._cuda(x, out)
        ops._req(x.dtype == torch.bfloat16 and x.shape[-1] == self.switch_mlp.hidden, "MoeBlock: bf16 x [.., hidden]")
        T = x.numel() // x.shape[-1]
        if out is None:
            out = torch.empty_like(x)
        ops._req(out.dtype == x.dtype and out.shape == x.shape, "MoeBlock: out must match x")
        aux_c, aux = None, None
        if return_aux:
            n, E, dev = T * self.top_k, self.switch_mlp.n_experts, x.device
            aux = dict(indices=torch.empty((T, self.top_k), dtype=torch.int32, device=dev),
                       scores=torch.empty((T, self.top_k), dtype=torch.bfloat16, device=dev),
                       perm=torch.empty(n, dtype=torch.int32, device=dev),
                       inv_perm=torch.empty(n, dtype=torch.int32, device=dev),
                       counts=torch.empty(E, dtype=torch.int32, device=dev),
                       offsets=torch.empty(E + 1, dtype=torch.int32, device=dev),
                       logits=torch.empty((T, E), dtype=torch.bfloat16, device=dev),
                       out_f32=torch.empty(x.shape, dtype=torch.float32, device=dev))
            aux_c = L.MoeAux(*[aux[n_].data_ptr() for n_ in ("indices", "scores", "perm", "inv_perm", "counts",
                                                             "offsets", "logits", "out_f32")])
        L.check(L.lib().b200_moe_block_forward(ops._ctx(self.ctx), C.byref(self._cfg), C.byref(self._params), L.ptr(x),
                                               T, L.ptr(out), C.byref(aux_c) if aux_c is not None else None,
                                               L.stream_ptr()))
        return (out, aux) if return_aux else out


def _forward_prenorm(self, x, residual=None, weight=None, eps=1e-5, out=None):
    """out = block(rms_norm(x + residual, weight, eps)) in one library call -> (x + residual or x itself, out):
    the pre-norm MLP half of a transformer layer (mlx-lm/src/models/qwen3.rs:310-325)."""
    ops._cuda(x, residual, weight, out)
    ops._req(x.dtype == torch.bfloat16 and x.shape[-1] == self.switch_mlp.hidden, "MoeBlock: bf16 x [.., hidden]")
    ops._req(residual is None or (residual.shape == x.shape and residual.dtype == x.dtype), "residual must match x")
    T = x.numel() // x.shape[-1]
    if out is None:
        out = torch.empty_like(x)
    s = torch.empty_like(x) if residual is not None else None
    L.check(L.lib().b200_moe_block_forward_prenorm(ops._ctx(self.ctx), C.byref(self._cfg), C.byref(self._params), L.ptr(x),
                                                   L.ptr(residual), L.ptr(weight), float(eps), T, L.ptr(s), L.ptr(out), None,
                                                   L.stream_ptr()))
    return (s if s is not None else x), out


MoeBlock.forward_prenorm = _forward_prenorm


def router_topk(x, gate_weight, top_k, router_mode=ROUTER_SOFTMAX_TOPK, norm_topk_prob=True, logit_bias=None,
                return_logits=False, ctx=None):
    """Router alone -> (indices [T,k] int32, scores [T,k] bf16[, logits [T,E] bf16])."""
    ops._cuda(x, gate_weight, logit_bias)
    T, H = x.numel() // x.shape[-1], x.shape[-1]
    E = gate_weight.shape[0]
    cfg = L.MoeConfig(H, 64, E, top_k, 4, 64, router_mode, int(norm_topk_prob))
    idx = torch.empty((T, top_k), dtype=torch.int32, device=x.device)
    sc = torch.empty((T, top_k), dtype=torch.bfloat16, device=x.device)
    lg = torch.empty((T, E), dtype=torch.bfloat16, device=x.device) if return_logits else None
    L.check(L.lib().b200_router_topk(ops._ctx(ctx), C.byref(cfg), L.ptr(x), L.ptr(gate_weight), L.ptr(logit_bias), T,
                                     L.ptr(idx), L.ptr(sc), L.ptr(lg), L.stream_ptr()))
    return (idx, sc, lg) if return_logits else (idx, sc)


class HostPipeline:
    """Serves a block (anything with forward(x, out=...)) from HOST memory.  Each `submit(x_host,
    out_host)` (pinned bf16 buffers [T, H]) uploads its input, runs the block and downloads the result;
    successive submits are software-pipelined on three streams - the upload of call i+1 overlaps the
    compute of call i and the download of call i-1 - with `depth` pairs of device buffers.  `submit`
    returns a ticket; `wait(ticket)` blocks until that call's output is in its host buffer, `drain()`
    until all are.  Results are those of block.forward on the same rows (same kernels, same order)."""

    def __init__(self, block, max_tokens, hidden, device, depth=2):
        self.block, self.depth = block, depth
        self.up, self.run, self.down = (torch.cuda.Stream(device=device) for _ in range(3))
        self.xd = [torch.empty((max_tokens, hidden), dtype=torch.bfloat16, device=device) for _ in range(depth)]
        self.od = [torch.empty((max_tokens, hidden), dtype=torch.bfloat16, device=device) for _ in range(depth)]
        self.ev_up = [torch.cuda.Event() for _ in range(depth)]
        self.ev_run = [torch.cuda.Event() for _ in range(depth)]
        self.ev_down = [torch.cuda.Event() for _ in range(depth)]
        self.n = 0

    def submit(self, x_host, out_host):
        ops._req(x_host.is_pinned() and out_host.is_pinned(), "HostPipeline: pinned host buffers")
        T = x_host.shape[0]
        ops._req(T <= self.xd[0].shape[0], "HostPipeline: more tokens than max_tokens")
        s = self.n % self.depth
        first = self.n < self.depth
        xd, od = self.xd[s][:T], self.od[s][:T]
        if self.n == 0:
            for st in (self.up, self.run, self.down):
                st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.up):
            if not first:
                self.up.wait_event(self.ev_run[s])     # the call that last read this input slot has run
            xd.copy_(x_host, non_blocking=True)
            self.ev_up[s].record(self.up)
        with torch.cuda.stream(self.run):
            self.run.wait_event(self.ev_up[s])
            if not first:
                self.run.wait_event(self.ev_down[s])   # this output slot has been downloaded
            self.block.forward(xd, out=od)
            self.ev_run[s].record(self.run)
        with torch.cuda.stream(self.down):
            self.down.wait_event(self.ev_run[s])
            out_host.copy_(od, non_blocking=True)
            self.ev_down[s].record(self.down)
        self.n += 1
        return s

    def wait(self, ticket):
        self.ev_down[ticket].synchronize()

    def drain(self, stream=None):
        """Make `stream` (default: the current one) wait for everything submitted so far."""
        stream = stream or torch.cuda.current_stream()
        for st in (self.up, self.run, self.down):
            stream.wait_stream(st)


class MoeStack:
    """A stack of pre-norm MoE blocks with residual connections and no attention (BASELINE.json
    configs[2]): per layer  h <- h + block(rms_norm(h, weight, eps)), the wiring of a transformer
    block's MLP half (mlx-lm/src/models/qwen3.rs:310-325) with the MLP replaced by the routed block.
    The residual add of layer l is fused with the norm of layer l+1 and handed to the block's entry point
    (`b200_moe_block_forward_prenorm`)."""

    def __init__(self, blocks, norm_weights=None, eps=1e-6, ctx=None):
        self.blocks, self.eps, self.ctx = list(blocks), eps, ctx
        self.norm_weights = list(norm_weights) if norm_weights is not None else [None] * len(self.blocks)

    def forward(self, x):
        h = x
        y = None
        for blk, w in zip(self.blocks, self.norm_weights):
            if hasattr(blk, "forward_prenorm"):
                # residual add of the previous layer, this layer's norm and the block: one library call
                h, y = blk.forward_prenorm(h, y, w, self.eps)
                continue
            # any other block with a forward(x) (the expert-parallel block): norm kernel, then the block
            if y is None:
                normed = ops.rms_norm(h, w, self.eps, ctx=self.ctx)
            else:
                h, normed = ops.add_rms_norm(h, y, w, self.eps, ctx=self.ctx)
            y = blk.forward(normed)
        out = torch.empty_like(h)
        L.check(L.lib().b200_add(ops._ctx(self.ctx), L.ptr(h), L.ptr(y), h.numel(), L.ptr(out), L.stream_ptr()))
        return out
