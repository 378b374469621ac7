"""Several mixers side by side: all read the same input, and the result is a constant times the sum of their outputs,
each first RMS-normed over the model width with a plain weight of its own,
    out = scale * sum_b rmsnorm(branch_b(x)) * w_b.
Each branch writes its output into a 32-bit buffer (Mixer.forward with overwrite=True); one kernel norms the buffers
and adds the sum into the residual.  A branch may be any registered mixer: it gets its own part of the schedule
entry's cache (the pages if it asked for pages, its own run of the fixed-size states).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..config.spec import ParamSpec, bundle_requirements, split_requirement
from ..registry import build_part
from .base import Mixer


class SideBySide(Mixer):
    def __init__(self, spec, env):
        super().__init__(spec, env)
        if not 1 <= len(spec.branches) <= 4:
            raise ValueError("one to four branches")
        self.names = [name for name, _ in spec.branches]
        self.branches = [build_part(branch, env) for _, branch in spec.branches]
        self.out_weights = [None] * len(self.branches)
        # which part of the entry's cache each branch sees: (pages?, first state, states)
        self.cache_parts, cursor = [], 0
        for branch in self.branches:
            pages, states = split_requirement(branch.cache_requirement())
            self.cache_parts.append((pages is not None, cursor, len(states)))
            cursor += len(states)

    @property
    def graph_safe(self):
        return all(branch.graph_safe for branch in self.branches)

    @property
    def takes_normed_residual(self):
        return all(branch.takes_normed_residual for branch in self.branches)

    @property
    def portion_multiple(self):
        import math
        return math.lcm(*[max(1, int(branch.portion_multiple)) for branch in self.branches])

    def cache_requirement(self):
        return bundle_requirements([branch.cache_requirement() for branch in self.branches])

    def parameters(self):
        table = {}
        for name, branch in zip(self.names, self.branches):
            for local, param in branch.parameters().items():
                table[f"{name}.{local}"] = param
            table[f"{name}.{self.spec.out_tensor}"] = ParamSpec((self.spec.hidden_size,), init="ones", store="float32")
        return table

    def bind(self, tensors):
        for index, (name, branch) in enumerate(zip(self.names, self.branches)):
            prefix = name + "."
            mine = {local[len(prefix):]: tensor for local, tensor in tensors.items() if local.startswith(prefix)}
            self.out_weights[index] = mine.pop(self.spec.out_tensor).contiguous()
            branch.bind(mine)

    def weight_bytes(self):
        return sum(branch.weight_bytes() for branch in self.branches) + sum(w.numel() * 4 for w in self.out_weights)

    def forward(self, ctx, cache, x, residual, overwrite=False):
        if overwrite:
            residual.zero_()
        outputs = []
        for branch, (pages, first, count) in zip(self.branches, self.cache_parts):
            out = ctx.alloc(tuple(residual.shape), torch.float32)
            branch.forward(ctx, cache.part(pages, first, count) if cache is not None else None, x, out, overwrite=True)
            outputs.append(out)
        kernels.add_normed_branches(outputs, self.out_weights, residual, self.spec.eps, self.spec.scale)
        ctx.residual_stats = None
