"""Mixture-of-experts feed-forward with a softmax router.

    p = softmax(Wr x) over all experts; the top-k p, in descending order, are the
    weights (divided by their sum if ``norm_topk_prob``);
    y = sum_k w_k * down_e( silu(gate_e x) * (up_e x) ), summed in rank order;
    y += sigmoid(w_sg . x) * shared(x)   (the gate only if the checkpoint has it).

Reference: router crates/ferrox-moe/src/lib.rs:333-355, expert :619-659, combine
:735-752, shared expert and its sigmoid gate crates/ferrox-models/src/decoder.rs:
2660-2681 and (batched) :1037-1093; tokens bucketed by expert :2792-2890.

Tokens are sorted by expert on the device (no host round trip between the router
and the experts); each expert's rows form one group of a grouped matrix product.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorDecl
from .base import FeedForward, register_part
from .mlp import pack_gate_up

# From this many tokens on the routed experts go through the tcgen05 kernel with swapped roles (measured).
SWAP_MIN_TOKENS = 8


def expert_tile_tokens(T: int, K: int, E: int):
    """Tokens per tile of the swapped-role kernel for the routed experts' products, by the mean number of rows
    an expert gets; None where the 128-row tiles of the plain tcgen05 kernel are as good.  Measured on a B200
    with 60 experts: decode batches of 8 to 64 tokens gain 5 to 25 %; with uniform routing the swapped kernel
    stays a few per cent ahead up to some 20 rows an expert, but routing is never uniform, an expert with more
    rows than a tile holds streams its matrix again for each further tile, and inside the model prompts of 512
    and 2048 tokens were faster with the 128-row tiles."""
    r = T * K / max(E, 1)
    if r <= 8:
        return 32, 32
    if r <= 16:
        return 64, 64
    return None




class SoftmaxTopkMoe(FeedForward):
    graph_safe = True
    fuses_norm = True
    def tensor_decls(self):
        s, p = self.spec, self.spec.prefix
        d = [TensorDecl(p + "gate.weight", (s.n_experts, s.hidden))]
        for e in range(s.n_experts):
            d += [
                TensorDecl(p + f"experts.{e}.gate_proj.weight", (s.expert_intermediate, s.hidden)),
                TensorDecl(p + f"experts.{e}.up_proj.weight", (s.expert_intermediate, s.hidden)),
                TensorDecl(p + f"experts.{e}.down_proj.weight", (s.hidden, s.expert_intermediate)),
            ]
        if s.shared_intermediate > 0:
            d += [
                TensorDecl(p + "shared_expert.gate_proj.weight", (s.shared_intermediate, s.hidden)),
                TensorDecl(p + "shared_expert.up_proj.weight", (s.shared_intermediate, s.hidden)),
                TensorDecl(p + "shared_expert.down_proj.weight", (s.hidden, s.shared_intermediate)),
            ]
            if s.shared_gate:
                d.append(TensorDecl(p + "shared_expert_gate.weight", (1, s.hidden), optional=True))
        return d

    def load(self, src, rt):
        super().load(src, rt)
        s, p = self.spec, self.spec.prefix
        self.w_router = src.get(p + "gate.weight")
        E, I, H = s.n_experts, s.expert_intermediate, s.hidden
        # If any expert tensor is stored in 32 bits, the packed buffers are 32-bit.
        names = [p + f"experts.{e}.{n}_proj.weight" for e in range(E) for n in ("gate", "up", "down")]
        dt = torch.float32 if any(src.dtype_of(n) == torch.float32 for n in names) else rt.dtype
        self.w_gu = torch.empty(E, 2 * I, H, dtype=dt, device=rt.device)
        self.w_down = torch.empty(E, H, I, dtype=dt, device=rt.device)
        for e in range(E):
            self.w_gu[e, :I].copy_(src.get(p + f"experts.{e}.gate_proj.weight"))
            self.w_gu[e, I:].copy_(src.get(p + f"experts.{e}.up_proj.weight"))
            self.w_down[e].copy_(src.get(p + f"experts.{e}.down_proj.weight"))
        self.w_shared_gu = self.w_shared_down = self.w_shared_gate = None
        if s.shared_intermediate > 0:
            self.w_shared_gu = pack_gate_up(
                src.get(p + "shared_expert.gate_proj.weight"), src.get(p + "shared_expert.up_proj.weight")
            )
            self.w_shared_down = src.get(p + "shared_expert.down_proj.weight")
            if s.shared_gate and src.has(p + "shared_expert_gate.weight"):
                self.w_shared_gate = src.get(p + "shared_expert_gate.weight").reshape(1, H).contiguous()
        # router rows and the shared expert's gate row share one product: [E (+1), H]
        self.w_route = self.w_router
        if self.w_shared_gate is not None:
            dtr = torch.float32 if torch.float32 in (self.w_router.dtype, self.w_shared_gate.dtype) else self.w_router.dtype
            self.w_route = torch.cat([self.w_router.to(dtr), self.w_shared_gate.to(dtr)], dim=0).contiguous()
        self._scratch = torch.zeros(2 * E, dtype=torch.int32, device=rt.device)
        if self.w_shared_gu is not None and rt.device.type == "cuda":
            self._side = torch.cuda.Stream(device=rt.device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()

    def _shared_expert(self, x, batch, st):
        """silu(gate) * up, then down, of the expert that every token visits: [T, H]."""
        s, rt = self.spec, self.rt
        T, Is = x.shape[0], s.shared_intermediate
        sact = rt.empty(T, Is)
        ops.gated_linear(x, self.w_shared_gu, sact, status=batch.status, stream=st)
        shared = rt.empty(T, s.hidden)
        ops.linear(sact, self.w_shared_down, shared, status=batch.status, stream=st)
        return shared

    def _shared_on_side(self, x, batch):
        """The shared expert's two products on the second stream, from the point the fork event marks."""
        self._side.wait_event(self._fork)
        with torch.cuda.stream(self._side):
            out = self._shared_expert(x, batch, self._side.cuda_stream)
            self._join.record(self._side)
        return out

    def forward_add(self, x, h, batch, then_norm=None):
        s, rt, st = self.spec, self.rt, batch.stream
        T, E, K, I, H = x.shape[0], s.n_experts, s.top_k, s.expert_intermediate, s.hidden
        i32 = torch.int32
        # A decode step of a few tokens: the router's product, the routing and the rows in expert order come from ONE
        # kernel (three dependent launches otherwise, each a few microseconds of waiting for the one before).
        fused = ops.route_fused_ok(x, self.w_route, E, K)
        tc = ops.tc_ok(x, self.w_gu) and I % 8 == 0 and E <= ops.TC_MAX_GROUPS
        tiles = expert_tile_tokens(T, K, E) if tc and T >= SWAP_MIN_TOKENS and E <= ops.TC_SWAP_MAX_GROUPS else None
        small = tiles is None and T <= ops.SKINNY_MAX_TOKENS and ops.skinny_ok(x, self.w_gu) and I % 32 == 0
        big = T > ops.SKINNY_MAX_TOKENS and tc
        n_route = self.w_route.shape[0]      # E router logits, then the shared expert's gate logit if it has one
        # The shared expert's two products run on a second stream beside the routing and the routed experts; both
        # meet again at the combination.  In a decode step the routed experts' kernels leave most of the machine
        # idle; in a prompt the router's short kernels hide under the shared expert's products.  Measured on a
        # B200: 3 to 10 % of a decode step of 8 to 64 tokens, 14 % of a prompt portion of 256 tokens, 4 % at 2,048.
        shared = None
        overlap = self.w_shared_gu is not None

        if overlap:
            main = torch.cuda.current_stream()
            self._fork.record(main)          # the shared expert may start from here on
            if not fused:
                shared = self._shared_on_side(x, batch)
        logits = rt.empty(T, n_route, dtype=torch.float32)
        ids = rt.empty(T, K, dtype=i32)
        weights = rt.empty(T, K, dtype=torch.float32)
        offsets = rt.empty(E + 1, dtype=i32)
        src_token = rt.empty(T * K, dtype=i32)
        inv_perm = rt.empty(T * K, dtype=i32)
        active = rt.empty(min(E, T * K), dtype=i32) if small else None
        xp = None
        if fused:
            # The cluster's kernel goes first: it needs eight free SMs of one GPC at once, which it finds now and would
            # not find once the shared expert's weight-streaming kernels (enqueued right after it, waiting only for what
            # was before it) fill every SM.
            xp = rt.empty(T * K, H) if tiles is not None else None
            ops.route_fused(x, self.w_route, logits, K, s.norm_topk_prob, ids, weights, offsets, src_token, inv_perm, active,
                            n_experts=E, xp_out=xp, stream=st)
            if overlap:
                shared = self._shared_on_side(x, batch)
        elif T <= ops.ROUTE_SMALL_MAX_TOKENS and E <= ops.ROUTE_SMALL_MAX_EXPERTS:
            ops.linear(x, self.w_route, logits, status=batch.status, stream=st)
            ops.route_small(logits, K, s.norm_topk_prob, ids, weights, offsets, src_token, inv_perm, active,
                            n_experts=E, stream=st)
        else:
            ops.linear(x, self.w_route, logits, status=batch.status, stream=st)
            ops.route(logits, K, s.norm_topk_prob, ids, weights, self._scratch, offsets, src_token, inv_perm, active,
                      n_experts=E, stream=st)

        act = rt.empty(T * K, I)
        y = rt.empty(T * K, H)
        if tiles is not None:
            # a few rows for each expert: rows in expert order, then features in the lanes of the tensor-core tiles
            # and the expert's rows in their columns
            if xp is None:
                xp = rt.empty(T * K, H)
                ops.gather_rows(x, src_token, xp, stream=st)
            # (the offsets were written by the routing, before the gather: both products may fetch weights early;
            # when one kernel did both, the first product waits for it before it reads the offsets)
            ops.gemm_tc_swap(xp, self.w_gu, act, gated=True, group_offsets=offsets, tokens_per_tile=tiles[0],
                             weights_first=not fused, status=batch.status, stream=st)
            ops.gemm_tc_swap(act, self.w_down, y, group_offsets=offsets, tokens_per_tile=tiles[1],
                             weights_first=True, status=batch.status, stream=st)
        elif small:
            # very few tokens: every expert that was chosen is streamed once, gate/up fused with SiLU
            ops.gemm_skinny(x, self.w_gu, act, gated=True, x_rows=src_token, group_offsets=offsets,
                            active_groups=active, tokens_hint=T, stream=st)
            ops.gemm_skinny(act, self.w_down, y, group_offsets=offsets, active_groups=active, tokens_hint=T, stream=st)
        elif big:
            # many tokens: bring them into expert order once, then grouped tensor-core products
            xp = rt.empty(T * K, H)
            ops.gather_rows(x, src_token, xp, stream=st)
            ops.gemm_tc(xp, self.w_gu, act, gated=True, group_offsets=offsets, status=batch.status, stream=st)
            ops.gemm_tc(act, self.w_down, y, group_offsets=offsets, status=batch.status, stream=st)
        else:
            gu = rt.empty(T * K, 2 * I)
            ops.gemm(x, self.w_gu, gu, a_rows=src_token, group_offsets=offsets, stream=st)
            ops.silu_mul(gu, act, stream=st)
            ops.gemm(act, self.w_down, y, group_offsets=offsets, stream=st)

        gate_logit = None
        if self.w_shared_gu is not None:
            if overlap:
                main.wait_event(self._join)
            else:
                shared = self._shared_expert(x, batch, st)
            if self.w_shared_gate is not None:
                gate_logit = logits[:, E:]      # [T, 1] view with the logits' row stride
        # the combination applies the norm that follows it where that is an RMSNorm over rows it can hold
        rms = then_norm.as_rms() if then_norm is not None else None
        if rms is not None and ops.combine_norm_ok(h, y):
            out = rt.empty(T, H)
            return ops.moe_combine(h, y, inv_perm, weights, shared, gate_logit, stream=st, norm=(rms[0], rms[1], out))
        ops.moe_combine(h, y, inv_perm, weights, shared, gate_logit, stream=st)
        return None


register_part("softmax_topk_moe", SoftmaxTopkMoe, replace=True)
