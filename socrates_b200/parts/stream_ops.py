"""Parts that act on the residual stream between layer runs (`RunEntry.before`).

"pass_inject": at the start of pass t over a group of repeated layers the stream gets a
learned vector `steps[t]` (tensor `<name>step`, [passes, d]) and, from the second pass on,
the embedding's output once more.  Nothing is computed here: the rows and the vector are
left on the stream and the next norm's kernel adds them with the pending branch, in one
pass over the residual.
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .base import ParamSpec, Part, ResidualStream, register_part


class PassInject(Part):
    def __init__(self, spec, name):
        super().__init__(spec, name)
        self.dim = int(spec.params["dim"])
        self.passes = int(spec.params["passes"])
        self.index = int(spec.params["index"])
        self.add_embedding = bool(spec.params.get("add_embedding", self.index > 0))
        self.needs_embedding_output = self.add_embedding
        self.steps: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        return {self.name + "step": ParamSpec((self.passes, self.dim), role="gain", init="normal")}

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype) -> None:
        self.steps = tensors[self.name + "step"]

    def apply(self, ctx, stream: ResidualStream) -> None:
        if stream.add_rows is not None or stream.add_vec is not None:
            raise RuntimeError("two stream ops in a row: the first one's additions are still waiting")
        stream.add_vec = self.steps[self.index]
        if self.add_embedding:
            stream.add_rows = stream.embedding_output


register_part("stream_op", "pass_inject", PassInject)
