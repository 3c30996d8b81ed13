"""Attention over a cached latent (kernels: csrc/latent_attention.cu).

Per token the mixer projects to ``[query latent | key/value latent | shared rotated key part]`` in
one product; the preparation kernel RMS-norms the two latents (32-bit), rotates the shared key
part and writes ``[c | k_rot]`` into the token's page slot: that row is all the cache holds.
Queries ``q = W_uq c_q`` are laid out head by head as ``[head_dim unrotated | rot_dim rotated]``.

Keys and values are never formed.  With ``k_plain = W_uk c`` and ``v = W_uv c``,

    q_plain . k_plain = (W_uk^T q_plain) . c          and        sum_j p_j v_j = W_uv (sum_j p_j c_j),

so the unrotated queries are taken into the latent's space (one batched product over the heads),
attention runs over the cached rows as if there were one key/value head of ``kv_rank + rot_dim``
dims whose first ``kv_rank`` dims are also the values, and the values' up-projection follows (one
more batched product).  Scores, weights and sums are 32-bit; the products are in the activation
type with 32-bit accumulation.
"""
from __future__ import annotations

import torch

from ..config.specs import ParamSpec
from ..csrc import ops
from .base import KVRequest, Mixer, make_position, register_mixer
from .linear import linear
from .position import as_rotary_args


class LatentAttention(Mixer):
    graph_safe = True
    max_step_entries = ops.LIMITS["grid_dim_yz"]

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        s = spec
        if min(s.hidden_size, s.num_heads, s.head_dim, s.v_head_dim, s.q_rank, s.kv_rank) <= 0 or s.rot_dim < 0:
            raise ValueError("the sizes of a latent attention must be positive (rot_dim may be 0)")
        if s.kv_rank + s.rot_dim > ops.LIMITS["latent_max_row"]:
            raise ValueError(f"a cached row of {s.kv_rank} + {s.rot_dim} elements is not supported (at most "
                             f"{ops.LIMITS['latent_max_row']}: a warp keeps a row in registers)")
        if s.num_heads > ops.LIMITS["grid_dim_yz"]:
            raise ValueError(f"{s.num_heads} heads are not supported (heads are a grid dimension of the kernels)")
        if s.window is not None and s.window <= 0:
            raise ValueError("window must be positive (None: all keys)")
        self.position = make_position(s.position, dtype) if s.position is not None and s.rot_dim > 0 else None
        if self.position is not None:
            if s.position.pairing != "split_half":
                raise ValueError("the latent attention kernels rotate split halves only")
            if s.position.rotary_dim > s.rot_dim:
                raise ValueError(f"the position encoding rotates {s.position.rotary_dim} dims, the rotated part has {s.rot_dim}")
        self.sink = None

    def parameters(self):
        s = self.spec
        out = {"down": ParamSpec((s.q_rank + s.kv_rank + s.rot_dim, s.hidden_size)),
               "q_norm": ParamSpec((s.q_rank,), "act", "norm"),
               "kv_norm": ParamSpec((s.kv_rank,), "act", "norm"),
               "uq": ParamSpec((s.num_heads * (s.head_dim + s.rot_dim), s.q_rank)),
               "uk": ParamSpec((s.num_heads * s.head_dim, s.kv_rank)),
               "uv": ParamSpec((s.num_heads * s.v_head_dim, s.kv_rank)),
               "o": ParamSpec((s.hidden_size, s.num_heads * s.v_head_dim))}
        if s.sink:
            out["sink"] = ParamSpec((s.num_heads,), "float32", "bias")
        return out

    def kv_request(self):
        s = self.spec
        return KVRequest(1, s.kv_rank + s.rot_dim, s.window, None, "latent")

    def forward(self, x, step, slot):
        s = self.spec
        tokens, dev = x.shape[0], x.device
        H, d, r, rank = s.num_heads, s.head_dim, s.rot_dim, s.kv_rank
        if self.position is not None:
            rope = as_rotary_args(self.position.kernel_args(dev))
            if rope.scale != 1.0:
                raise ValueError("the latent attention kernels take no factor on cos and sin")
            inv_freq, rotary_dim = rope.inv_freq, rope.rotary_dim
        else:
            inv_freq, rotary_dim = None, 0
        proj = linear(x, self.down)
        cq = torch.empty(tokens, s.q_rank, dtype=x.dtype, device=dev)
        ops.latent_prep(proj, self.q_norm, self.kv_norm, inv_freq, step.positions, step.token_seq, step.seq_rows,
                        slot.table, slot.kv, cq, q_rank=s.q_rank, rank=rank, rot=r, rotary_dim=rotary_dim,
                        eps=s.norm_eps, page_size=slot.page_size, write_cache=slot.write_cache)
        q = linear(cq, self.uq)                                              # [tokens, H * (d + r)]
        # the unrotated queries in the latent's space: [H, tokens, d] x [H, d, rank], 32-bit out
        q_plain = q.view(tokens, H, d + r)[:, :, :d].transpose(0, 1)
        q_lat = torch.bmm(q_plain, self.uk.view(H, d, rank), out_dtype=torch.float32) if x.dtype != torch.float32 \
            else torch.bmm(q_plain, self.uk.view(H, d, rank))
        out_lat = torch.empty(tokens, H, rank, dtype=x.dtype, device=dev)
        self.attend(q_lat, q, inv_freq, rotary_dim, out_lat, step, slot)
        # the values' up-projection per head, read from and written to token-major rows through strided views
        heads_out = torch.empty(tokens, H, s.v_head_dim, dtype=x.dtype, device=dev)
        torch.bmm(out_lat.transpose(0, 1), self.uv.view(H, s.v_head_dim, rank).transpose(1, 2), out=heads_out.transpose(0, 1))
        return linear(heads_out.view(tokens, H * s.v_head_dim), self.o)

    use_tensor_cores = None      # False: always the kernel with one block per (token, head)

    def attend(self, q_lat, q, inv_freq, rotary_dim, out_lat, step, slot):
        """bfloat16 steps of sizes the tiled kernel takes (latent and rotated part in multiples of 16, a
        cached row of at most 256) run on tensor-core tiles whose rows are (token, head) pairs, prompt
        portions and single tokens alike; everything else one block per (token, head)."""
        s = self.spec
        if (self.use_tensor_cores is not False and q.dtype == torch.bfloat16 and s.scale > 0
                and ops.latent_attention_tiled_supported(s.kv_rank, s.rot_dim)):
            qfull = torch.empty(q.shape[0], s.num_heads, s.kv_rank + s.rot_dim, dtype=q.dtype, device=q.device)
            ops.latent_q_pack(q_lat, q, inv_freq, step.positions, qfull, heads=s.num_heads, head_dim=s.head_dim,
                              rank=s.kv_rank, rot=s.rot_dim, rotary_dim=rotary_dim)
            ops.latent_attention_tiled(qfull, slot.kv, slot.table, step.seq_rows, step.cu_q, step.kv_len, self.sink,
                                       out_lat, entries=step.num_seqs, max_q_len=step.max_q_len, heads=s.num_heads,
                                       rank=s.kv_rank, rot=s.rot_dim, page_size=slot.page_size, scale=s.scale,
                                       window=s.window,
                                       max_keys=step.max_kv_len if s.window is None else min(step.max_kv_len, s.window + step.max_q_len - 1))
            return
        ops.latent_attention_plain(q_lat, q, inv_freq, slot.kv, slot.table, step.seq_rows, step.token_seq,
                                   step.positions, self.sink, out_lat, heads=s.num_heads, head_dim=s.head_dim,
                                   rank=s.kv_rank, rot=s.rot_dim, rotary_dim=rotary_dim, page_size=slot.page_size,
                                   scale=s.scale, window=s.window)


register_mixer("latent_attention", LatentAttention)
