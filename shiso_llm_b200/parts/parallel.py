"""Several mixers side by side on the same input: ``sum_b scale_b * mixer_b(h)``.

Every branch is a mixer that can work on columns: it has ``in_matrix`` (its input
projections joined, ``[in_width, hidden]``), ``mix(proj, step, cache, out, out_scale)`` and
``out_matrix`` (``[hidden, out_width]``).  The branches' input matrices are joined into ONE
product over ``h``, each branch reads its columns of the result and writes its columns of
one joint buffer - already multiplied by its scale, in float32 before rounding - and the
output projections, joined along their inputs, are ONE product that adds the branches up.
A branch's cache needs are the mixer's, in the branches' order.
"""

from __future__ import annotations

import torch

from .base import MIXERS, DeferredLinear, Mixer, project


@MIXERS.register("parallel_mixer")
class ParallelMixer(Mixer):
    """``params``: ``branches``, a list of ``(PartSpec, scale)``."""

    takes_deferred_norm = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.branches = [MIXERS.build(part, env) for part, _ in spec.params["branches"]]
        self.scales = [float(scale) for _, scale in spec.params["branches"]]
        for branch in self.branches:
            if not all(hasattr(branch, a) for a in ("mix", "in_width", "out_width")):
                raise ValueError(f"{type(branch).__name__} cannot work on the columns of a joint product")
        self.in_matrix = self.out_matrix = None
        # where each branch's views lie in the tuple this mixer is handed
        self._needs, self._cache_slices = [], []
        for branch in self.branches:
            need = branch.cache_spec()
            members = list(need) if isinstance(need, (tuple, list)) else ([] if need is None else [need])
            self._cache_slices.append((len(self._needs), len(members), isinstance(need, (tuple, list))))
            self._needs += members

    def sub_parts(self):
        return list(self.branches)

    def tensor_specs(self):
        return [spec for branch in self.branches for spec in branch.tensor_specs()]

    def bind(self, tensors):
        for branch in self.branches:
            branch.bind(tensors)
        ins = [b.in_matrix for b in self.branches]
        outs = [b.out_matrix for b in self.branches]
        if len({m.dtype for m in ins + outs}) > 1:
            ins, outs = [m.float() for m in ins], [m.float() for m in outs]
        self.in_matrix = torch.cat(ins, dim=0).contiguous()
        self.out_matrix = torch.cat(outs, dim=1).contiguous()
        for branch in self.branches:  # the joint matrices stand for them
            branch.in_matrix = branch.out_matrix = None

    def cache_spec(self):
        return tuple(self._needs)

    def forward(self, x, step, cache):
        ops = self.env.ops
        proj = project(ops, x, self.in_matrix, self.env.dtype)
        out = torch.empty((proj.shape[0], self.out_matrix.shape[1]), dtype=self.env.dtype, device=proj.device)
        col_in = col_out = 0
        for branch, scale, (first, count, is_tuple) in zip(self.branches, self.scales, self._cache_slices):
            view = tuple(cache[first : first + count]) if is_tuple else (cache[first] if count else None)
            branch.mix(proj[:, col_in : col_in + branch.in_width], step, view, out[:, col_out : col_out + branch.out_width], scale)
            col_in += branch.in_width
            col_out += branch.out_width
        return DeferredLinear(ops, out, self.out_matrix, self.env.dtype)
