"""Feed-forwards beside the gated one of ``parts/standard.py``.

=============  ======================  ==========================================
category       kind                    params
=============  ======================  ==========================================
ffn            ``none``                — (a layer without a feed-forward)
ffn            ``mlp``                 width, intermediate, activation
                                       (``relu2``: the square of relu),
                                       names (up, down -> local names)
ffn            ``table_moe``           width, vocab, experts, top, intermediate,
                                       shared (PartSpec of a feed-forward that
                                       runs for every token, or None),
                                       names (expert: a pattern with ``{i}``,
                                       gate, up, down, table, shared: a prefix)
=============  ======================  ==========================================

``table_moe``: a mixture of gated experts without a router.  An integer table
[vocab, top] names, for every token id, the ``top`` different experts that its tokens
use; each weighs 1/top.  Expert i is down_i(silu(gate_i h) * (up_i h)), no biases.
The result is the weighted sum of the chosen experts' results plus, if there is one,
the shared part's.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from .. import ops
from .base import FeedForward, TensorSpec, build_part, register_part
from .linear import Linear


class NoFeedForward(FeedForward):
    PROMPT_CAPTURABLE = True
    IS_NONE = True

    def forward(self, x, batch):
        return torch.zeros((1,) + tuple(x.shape), dtype=torch.float32, device=x.device)


class MLP(FeedForward):
    """down(act(up x)), no biases."""

    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.width, self.intermediate = int(params["width"]), int(params["intermediate"])
        self.activation = str(params.get("activation", "relu2"))
        if self.activation != "relu2":
            raise ValueError(f"unsupported activation {self.activation} (relu2)")
        names = dict(up="up_proj.weight", down="down_proj.weight")
        names.update(params.get("names") or {})
        self.names = names
        self.up = Linear(self.intermediate, self.width, ctx)
        self.down = Linear(self.width, self.intermediate, ctx)

    def tensor_specs(self):
        return [TensorSpec(self.names["up"], (self.intermediate, self.width)),
                TensorSpec(self.names["down"], (self.width, self.intermediate))]

    def load(self, fetch):
        self.up.load_rows([fetch(self.names["up"])])
        self.down.load_rows([fetch(self.names["down"])])

    def tensor(self, name):
        if name == self.names["up"]:
            return self.up.rows(0, self.intermediate)
        return self.down.rows(0, self.width) if name == self.names["down"] else None

    def weight_bytes(self):
        return self.up.weight_bytes() + self.down.weight_bytes()

    def forward(self, x, batch):
        a = ops.relu_squared_(self.up.forward(x, self.ctx.dtype))
        return self.down.forward_delta(a)


class TableMoE(FeedForward):
    PROMPT_CAPTURABLE = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        p = params
        self.width, self.vocab = int(p["width"]), int(p["vocab"])
        self.experts, self.top, self.intermediate = int(p["experts"]), int(p["top"]), int(p["intermediate"])
        if not 0 < self.top <= self.experts:
            raise ValueError(f"{self.top} of {self.experts} experts per token")
        names = dict(expert="experts.{i}.", gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight",
                     table="table", shared="shared.")
        names.update(p.get("names") or {})
        self.names = names
        shared = p.get("shared")
        self.shared = build_part("ffn", shared, ctx) if shared is not None else None
        self.PROMPT_CAPTURABLE = self.shared is None or bool(self.shared.PROMPT_CAPTURABLE)
        self.gate_up: Optional[torch.Tensor] = None      # [experts, 2, intermediate, width]
        self.down: Optional[torch.Tensor] = None         # [experts, width, intermediate]
        self.table: Optional[torch.Tensor] = None        # int32 [vocab, top]
        self.up_tiles: Optional[torch.Tensor] = None     # the experts' gate/up and down matrices as tiles (bfloat16)
        self.down_tiles: Optional[torch.Tensor] = None

    def _expert(self, i: int, which: str) -> str:
        return self.names["expert"].format(i=i) + self.names[which]

    def tensor_specs(self):
        f, w = self.intermediate, self.width
        specs = []
        for i in range(self.experts):
            specs += [TensorSpec(self._expert(i, "gate"), (f, w)), TensorSpec(self._expert(i, "up"), (f, w)),
                      TensorSpec(self._expert(i, "down"), (w, f))]
        specs.append(TensorSpec(self.names["table"], (self.vocab, self.top), "table", init="distinct_below",
                                init_arg=self.experts))
        if self.shared is not None:
            specs += [TensorSpec(self.names["shared"] + s.name, s.shape, s.role, s.optional, s.init, s.init_arg)
                      for s in self.shared.tensor_specs()]
        return specs

    def load(self, fetch):
        hold = self.ctx.hold
        self.gate_up = torch.stack([torch.stack([hold(fetch(self._expert(i, "gate")), "matrix"),
                                                 hold(fetch(self._expert(i, "up")), "matrix")]) for i in range(self.experts)])
        self.down = torch.stack([hold(fetch(self._expert(i, "down")), "matrix") for i in range(self.experts)])
        self.table = hold(fetch(self.names["table"]), "table")
        self.table_host = self.table.cpu().numpy()
        lo, hi = int(self.table_host.min()), int(self.table_host.max())
        if lo < 0 or hi >= self.experts:
            raise ValueError(f"the expert table names expert {lo if lo < 0 else hi}; there are {self.experts}")
        if self.shared is not None:
            self.shared.load(lambda n: fetch(self.names["shared"] + n))
        # The same matrices once more, as tiles for the tensor-core product of steps with many tokens
        # (bfloat16; rows of 16-byte multiples): all experts one after the other in one operand.
        self.up_tiles = self.down_tiles = None
        if (self.ctx.dtype == torch.bfloat16 and self.gate_up.is_cuda and not ops.plain_kernels()
                and self.width % 8 == 0 and self.intermediate % 8 == 0):
            from ..ops import gemm_tc
            self.up_tiles = torch.cat([gemm_tc.pack(self.gate_up[i].reshape(2 * self.intermediate, self.width), gated=True)
                                       for i in range(self.experts)], 0)
            self.down_tiles = torch.cat([gemm_tc.pack(self.down[i]) for i in range(self.experts)], 0)

    def tensor(self, name):
        for i in range(self.experts):
            pre = self.names["expert"].format(i=i)
            if name.startswith(pre):
                which = name[len(pre):]
                if which == self.names["gate"]:
                    return self.gate_up[i, 0]
                if which == self.names["up"]:
                    return self.gate_up[i, 1]
                if which == self.names["down"]:
                    return self.down[i]
        if name == self.names["table"]:
            return self.table
        if self.shared is not None and name.startswith(self.names["shared"]):
            return self.shared.tensor(name[len(self.names["shared"]):])
        return None

    def weight_bytes(self):
        """What a step of one token reads: its experts and the shared part."""
        el = self.gate_up.element_size() if self.gate_up is not None else (2 if self.ctx.dtype == torch.bfloat16 else 4)
        n = self.top * 3 * self.intermediate * self.width * el
        return n + (self.shared.weight_bytes() if self.shared is not None else 0)

    def forward(self, x, batch):
        base = None
        if self.shared is not None:
            base = self.shared.forward(x, batch)
            if base.dim() == 2:
                base = base.unsqueeze(0)
        n = x.shape[0]
        if self.up_tiles is not None and n >= self.SORTED_FROM:
            return self._forward_sorted(x, batch, base)
        hidden = ops.moe_table_up(x, batch.tokens, self.table, self.gate_up)
        return ops.moe_table_down(hidden, batch.tokens, self.table, self.down, 1.0 / self.top, base).unsqueeze(0)

    # From this many tokens on a step sorts its rows by expert, every expert's rows starting at a
    # multiple of 256, and runs ONE tensor-core product over all of them: a tile of 256 rows is
    # multiplied with the matrices of the expert the tile belongs to.  How many rows that makes
    # depends on the step's tokens: the host counts them from the step's token ids where the step's
    # description has them (the table is a constant); otherwise (a captured step, whose tokens the
    # host never sees) the product runs over the most rows there can be, and the tiles beyond the
    # last expert's hold zeros.  Fewer tokens go through the kernels that walk the matrices by expert.
    SORTED_FROM = 16
    ROW_TILE = 256

    def _forward_sorted(self, x, batch, base):
        from ..ops import gemm_tc
        n, dt, pad = x.shape[0], self.ctx.dtype, self.ROW_TILE
        counts, row_of, tiles = ops.moe_route(batch.tokens, self.table, self.experts, pad=pad)
        host = getattr(batch, "host", None)
        if host is not None and not torch.cuda.is_current_stream_capturing():
            ids = host[batch.layout.tokens:batch.layout.tokens + n]
            counts = np.bincount(self.table_host[ids].ravel(), minlength=self.experts)
            rows = int(((counts + pad - 1) // pad * pad).sum())
        else:
            rows = min(self.experts, n * self.top) * pad + (n * self.top) // pad * pad
        f, w = self.intermediate, self.width
        f_pad, w_pad = (f + 127) // 128 * 128, (w + 127) // 128 * 128
        xs = ops.moe_gather(x, row_of, rows)
        hidden = torch.empty((rows, f), dtype=dt, device=x.device)
        y = torch.empty((rows, w), dtype=torch.float32, device=x.device)
        gemm_tc.gemm_tc_pair(xs, self.up_tiles, f, out=hidden, ldo=f, gated=True, pair_offset=f_pad, b_packed=True,
                             groups=tiles, group_rows=2 * f_pad)
        gemm_tc.gemm_tc_pair(hidden, self.down_tiles, w, out=y, ldo=w, b_packed=True, groups=tiles, group_rows=w_pad)
        return ops.moe_combine(y, row_of, 1.0 / self.top, base).unsqueeze(0)


register_part("ffn", "none", NoFeedForward)
register_part("ffn", "mlp", MLP)
register_part("ffn", "table_moe", TableMoE)
