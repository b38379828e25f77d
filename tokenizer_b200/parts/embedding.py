"""Token embedding and output head.  The head multiplies the wanted rows, after
the final norm, by its own matrix or by the embedding it is tied to; logits are
float32 (reference: qwen-infer/src/model.rs:693-697, 750-758, 1224-1242)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.store import TensorSpec
from .base import register_part
from .linear import Linear
from .norm import tensor_name


class TokenEmbedding:
    @staticmethod
    def tensors(spec):
        out = [TensorSpec(tensor_name(spec), (spec.params["vocab_size"], spec.params["hidden_size"]))]
        if spec.params.get("position_tensor"):
            out.append(TensorSpec(spec.params["position_tensor"], (spec.params["positions"], spec.params["hidden_size"])))
        return out

    def __init__(self, spec, store, runtime):
        self.runtime = runtime
        self.vocab, self.hidden = int(spec.params["vocab_size"]), int(spec.params["hidden_size"])
        self.table = runtime.matrix(store.get(tensor_name(spec)))
        # `position_tensor` (optional): a learned vector per position, [positions, hidden], added to the
        # looked-up row as it is (the model then says `wants_positions` and is handed the rows' positions)
        self.positions = None
        if spec.params.get("position_tensor"):
            self.positions = runtime.matrix(store.get(spec.params["position_tensor"]))
        self.wants_positions = self.positions is not None
        # `scale` (optional): the looked-up row is multiplied by it, in float32; a head tied to
        # the table uses the table itself, without it
        self.scale = float(spec.params.get("scale", 1.0))

    def forward(self, ids, pos=None, row_req=None):
        x = self.runtime.empty(ids.shape[0], self.hidden, dtype=torch.float32)
        if self.positions is not None:
            if pos is None or row_req is None:
                raise ValueError("this embedding adds a vector per position: it needs the rows' positions")
            ops.embed_positions(ids, pos, row_req, self.table, self.positions, x, self.scale)
        else:
            ops.embed(ids, self.table, x, self.scale)
        return x


class LMHead:
    @staticmethod
    def tensors(spec):
        if spec.params.get("tied_to"):
            return []
        return [TensorSpec(tensor_name(spec),
                           (spec.params["vocab_size"], spec.params["hidden_size"]))]

    def __init__(self, spec, store, runtime, tied_table=None):
        self.runtime = runtime
        if spec.params.get("tied_to"):
            if tied_table is None:
                raise ValueError("a tied head needs the embedding table")
            self.proj = Linear(tied_table)
        else:
            self.proj = Linear(runtime.matrix(store.get(tensor_name(spec))))

    def forward(self, h):
        return self.proj.forward(h, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
