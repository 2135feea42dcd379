"""Latent attention: keys and values of a token are one normed low-rank latent plus one rotated key
part that all heads share, and only those are cached.

Per token with input h: the query latent ``cq = rms(W_dq h) * w`` and the queries ``q = W_uq cq``, head by
head ``[dim plain | rot_dim rotated]``; ``W_dkv h`` gives the latent ``c = rms(first kv_rank) * w`` and the
key part ``r = rotate(last rot_dim)``.  Head h's key is ``[W_uk[h] c | r]``, its value ``W_uv[h] c``; scores
``(q_plain . k_plain + q_rot . r) * scale``, causal softmax, then the output projection.

The cache holds the row ``[c | r]`` per token: one key/value head of size ``kv_rank + rot_dim`` whose first
``kv_rank`` elements double as the value.  The key up-projection is absorbed into the query
(``q_plain . W_uk[h] c = (W_uk[h]^T q_plain) . c``) and the value up-projection applied after the
mixing (``sum_j p_j W_uv[h] c_j = W_uv[h] sum_j p_j c_j``), so attention runs on the cached rows as they
are, with every query head on the one cached head.

Where a cached row has 64 or 128 elements (bfloat16) the tensor-core attention kernels take it as key
and as value at once: the mixed rows then carry ``rot_dim`` elements more than the value up-projection
reads (a fifth to a quarter more work in the second product, none in memory traffic).  Other row
sizes, and the 32-bit path, run the general kernel, which reads the values out of the key rows.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.specs import TensorSpec
from .base import CacheView, Mixer, PagedKVNeed, StepContext, build_nested, register_part


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    @classmethod
    def tensor_specs(cls, spec):
        hidden, heads = spec["hidden_size"], spec["num_heads"]
        dim, rot, value = spec["head_size"], spec["rotary_size"], spec["value_head_size"]
        kv_rank, q_rank = spec["kv_rank"], spec["q_rank"]
        return {
            "q_down.weight": TensorSpec((q_rank, hidden)),
            "q_norm.weight": TensorSpec((q_rank,), "scale"),
            "q_up.weight": TensorSpec((heads * (dim + rot), q_rank)),
            "kv_down.weight": TensorSpec((kv_rank + rot, hidden)),
            "kv_norm.weight": TensorSpec((kv_rank,), "scale"),
            "k_up.weight": TensorSpec((heads * dim, kv_rank)),
            "v_up.weight": TensorSpec((heads * value, kv_rank)),
            "o_proj.weight": TensorSpec((hidden, heads * value)),
        }

    @classmethod
    def kernel_libraries(cls, spec, runtime):
        row = int(spec["kv_rank"]) + int(spec["rotary_size"])
        fast = (f"attention_tcgen05:HEAD_SIZE={row}",) if cls._row_on_tensor_cores(row, runtime.dtype) else ()
        return ("pointwise", "latent", "attention_generic", "gemm_simt") + \
            (("gemm_tcgen05",) if runtime.dtype == torch.bfloat16 else ()) + fast

    @staticmethod
    def _row_on_tensor_cores(row: int, dtype) -> bool:
        return dtype == torch.bfloat16 and row in (64, 128)

    def __init__(self, spec, tensors, runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.dim = int(spec["head_size"])
        self.rot_dim = int(spec["rotary_size"])
        self.value_size = int(spec["value_head_size"])
        self.kv_rank = int(spec["kv_rank"])
        self.q_rank = int(spec["q_rank"])
        self.scale = float(spec["scale"])
        self.eps = float(spec["eps"])
        self.row = self.kv_rank + self.rot_dim
        if self.row > ops.MAX_GENERIC_HEAD_SIZE:
            raise ops.UnsupportedSize(
                f"latent rows of {self.row} elements: the attention kernel takes up to {ops.MAX_GENERIC_HEAD_SIZE}")
        self.position = build_nested("position", spec["position"], tensors, runtime)
        if 2 * self.position.inv_freq.shape[0] != self.rot_dim:
            raise ValueError("the position encoding must rotate the whole rotated key part")
        heads = self.num_heads
        # one product for both down-projections: [query latent | kv latent | key part]
        self.down_weight = runtime.matrix(torch.cat([tensors["q_down.weight"], tensors["kv_down.weight"]], dim=0))
        self.q_norm = runtime.vector(tensors["q_norm.weight"])
        self.kv_norm = runtime.vector(tensors["kv_norm.weight"])
        self.q_up = runtime.matrix(tensors["q_up.weight"])
        # absorbed into the query: per head [kv_rank, dim], the transpose of the key up-projection
        k_up = tensors["k_up.weight"].reshape(heads, self.dim, self.kv_rank)
        self.k_up_t = runtime.matrix(k_up.transpose(1, 2).contiguous())
        self.v_up = runtime.matrix(tensors["v_up.weight"].reshape(heads, self.value_size, self.kv_rank))
        self.out_weight = runtime.matrix(tensors["o_proj.weight"])
        self.fast = self._row_on_tensor_cores(self.row, runtime.dtype)

    def launch_key(self, ctx: StepContext, page_size: int) -> tuple:
        """As for the attention mixer: the decode kernel's shape follows the batch and the longest context."""
        singles = int(ctx.single_tokens.shape[0])
        if not singles:
            return ()
        if not (self.fast and ops.has_tcgen05_attention(self.row, page_size)):
            # the shared-row decode kernel cuts a token's keys by the batch and the longest context
            return ("shares", ops.latent_decode_splits(singles, self.num_heads, ctx.max_context_len)) if ctx.decode_only else ()
        return ops.decode_plan(singles, self.num_heads, 1, self.row, page_size, ctx.max_context_len)

    def launch_group(self):
        return ("latent_attention", self.num_heads, self.row, self.fast)

    def cache_need(self):
        # the values are the first kv_rank elements of the rows: no value cache of its own
        return PagedKVNeed(1, self.row, None, 0)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        dtype, device = self.runtime.dtype, x.device
        heads = self.num_heads
        interleaved = getattr(self.position, "interleaved", False)
        down = ops.project(x, self.down_weight, ctx.status)
        q_latent = torch.empty((tokens, self.q_rank), dtype=dtype, device=device)
        writes = cache.writes and cache.k is not None
        ops.latent_down_store(
            down, self.q_rank, self.kv_rank, self.rot_dim, self.q_norm, self.kv_norm, self.eps, ctx.positions,
            self.position.inv_freq, interleaved, ctx.slots[cache.group] if writes else None, q_latent,
            cache.k if writes else None, ctx.status,
        )
        q = ops.project(q_latent, self.q_up, ctx.status)
        q_plain = torch.empty((tokens, heads, self.dim), dtype=dtype, device=device)
        q_full = torch.empty((tokens, heads, self.row), dtype=dtype, device=device)
        ops.latent_q_store(q, ctx.positions, self.position.inv_freq, interleaved, q_plain, q_full)
        ops.per_head_project(q_plain, self.k_up_t, q_full[:, :, : self.kv_rank])
        table = ctx.block_tables[cache.group]
        if self.fast and ops.has_tcgen05_attention(self.row, cache.k.shape[2]):
            # the cached rows are keys and values at once; the value up-projection reads the first kv_rank
            mixed_rows = torch.empty((tokens, heads, self.row), dtype=dtype, device=device)
            if ctx.single_tokens.shape[0]:
                ops.paged_decode_attention_auto(
                    q_full, cache.k, cache.k, table, ctx.seq_of_token, ctx.positions, mixed_rows, self.scale, None,
                    ctx.status, None if ctx.decode_only else ctx.single_tokens, max_context=ctx.max_context_len,
                )
            if ctx.q_tiles.shape[0]:
                ops.paged_prefill_attention(
                    q_full, cache.k, cache.k, table, ctx.q_tiles, mixed_rows, self.scale, None, ctx.status,
                    cached_before=ctx.max_portion_start,
                )
            mixed_latent = mixed_rows[:, :, : self.kv_rank]
        elif ctx.decode_only:
            # every token stands alone: sixteen heads a CTA share the rows it stages, the keys are cut in shares
            mixed_latent = torch.empty((tokens, heads, self.kv_rank), dtype=dtype, device=device)
            ops.latent_decode_attention(
                q_full, cache.k, table, ctx.seq_of_token, ctx.positions, mixed_latent, self.scale,
                ops.latent_decode_splits(tokens, heads, ctx.max_context_len), ctx.status,
            )
        else:
            mixed_latent = torch.empty((tokens, heads, self.kv_rank), dtype=dtype, device=device)
            ops.paged_attention_generic(
                q_full, cache.k, None, table, ctx.seq_of_token, ctx.positions, mixed_latent,
                self.scale, None, ctx.status, values_in_keys=self.kv_rank,
            )
        mixed = torch.empty((tokens, heads, self.value_size), dtype=dtype, device=device)
        ops.per_head_project(mixed_latent, self.v_up, mixed)
        return ops.project(mixed.view(tokens, -1), self.out_weight, ctx.status)
