"""Grouped-query attention over the paged cache (models/llama/common/src/compute.rs:210-270).

qkv = x1 Wqkv^T (one merged product, heads ordered q, k, v); rotary encoding of q and k fused with
the write of k and v into the cache; causal attention of the step's tokens over everything their
sequences hold; out = o Wo^T.  The residual sum is the caller's (the block's) business.
"""
from __future__ import annotations

import math

import torch

from ..csrc import lib
from .base import MIXERS, POSITIONS, CacheNeed, Mixer, ParamDecl
from .linear import matmul_nt
from .spec import PartSpec


USE_TCGEN05 = True     # prompts: the tcgen05 kernel before the mma.sync one
USE_DECODE_RING = True  # decoding: the kernel with a ring of cache pages (TMA, tensor cores) before the register-staged one
FUSE_DECODE_ROPE = True # decoding: that kernel also rotates q and k and writes the cache (no rotary kernel)
RING_BLOCKS_PER_SM = 2  # decoding: the keys are sliced until that kernel has this many blocks per SM


@MIXERS.register("attention")
class Attention(Mixer):
    """params: width, nh, nkvh, dh, position (a PartSpec of a rotary encoding, or None)."""

    def __init__(self, params, dtype, device):
        super().__init__(params, dtype, device)
        self.d = int(params["width"])
        self.nh = int(params["nh"])
        self.nkvh = int(params["nkvh"])
        self.dh = int(params["dh"])
        if self.nh % self.nkvh:
            raise ValueError(f"{self.nh} heads cannot share {self.nkvh} key/value heads")
        if self.dh % 16 or self.dh > 256:
            raise ValueError(f"the attention kernels take head sizes 16, 32, ..., 256; got {self.dh}")
        pos = params.get("position")
        self.position = POSITIONS.build(pos, dtype, device) if isinstance(pos, PartSpec) else None
        self.qkv_width = (self.nh + 2 * self.nkvh) * self.dh
        self.scale = 1.0 / math.sqrt(self.dh)
        # query tiles this mixer asks the step to plan: the general kernel's, and the prompt kernel's
        self.general_tile = lib.attention_tile_tokens(self.nh, self.nkvh)
        # bfloat16 prompts: the mma.sync kernel takes every head size, the tcgen05 kernel heads of 64 and 128
        self.prompt_tile = lib.attention_prefill_tile_tokens() if dtype == torch.bfloat16 else 0
        self.tc_tile = lib.attention_tc_tile_tokens() if (self.prompt_tile and self.dh in (64, 128)) else 0
        self.tile_sizes = [t for t in (self.general_tile, self.prompt_tile, self.tc_tile) if t]

    @property
    def graph_safe(self) -> bool:
        return self.position is None or self.position.graph_safe

    @property
    def launches_only(self) -> bool:
        return self.position is None or self.position.launches_only

    def parameters(self):
        decl = {
            "wqkv": ParamDecl((self.qkv_width, self.d)),
            "wo": ParamDecl((self.d, self.nh * self.dh)),
        }
        if self.position is not None:      # what the position encoding has learned travels with its mixer
            decl.update({"position." + n: d for n, d in self.position.parameters().items()})
        return decl

    def bind(self, tensors) -> None:
        super().bind(tensors)
        if self.position is not None:
            self.position.bind({n: tensors["position." + n] for n in self.position.parameters()})

    def cache_need(self):
        return CacheNeed("full", self.nkvh, self.dh)

    def forward(self, ctx, x1, out, cache, state) -> None:
        nt = x1.shape[0]
        sfx = lib.suffix(self.dtype)
        qkv = ctx.scratch("attn.qkv", (nt, self.qkv_width), self.dtype)
        matmul_nt(x1, self.weights["wqkv"], qkv)
        table = ctx.page_table(cache)
        rotation = self.position.rotation() if self.position is not None else None
        if rotation is not None:
            cos, sin, half = rotation      # a rotary encoding: fused with the cache write below
        else:
            if self.position is not None:
                self.position.apply(ctx, qkv, self.nh, self.nkvh, self.dh)     # any other: by its own means
            cos, sin = ctx.identity_rotation(self.dh)
            half = 0
        o = ctx.scratch("attn.o", (nt, self.nh * self.dh), self.dtype)
        if ctx.decode and self._decode_fused(ctx, qkv, o, cache, table, nt, cos, sin, half):
            matmul_nt(o, self.weights["wo"], out)      # rotation and cache write happened inside the attention kernel
            return
        kc, vc = (cache.k, cache.v) if cache.writable else (None, None)
        lib.call("tb_rope_cache_" + sfx, lib.ptr(qkv), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos),
                 lib.ptr(table), ctx.max_pages, lib.ptr(cos), lib.ptr(sin), lib.ptr(kc), lib.ptr(vc),
                 nt, self.nh, self.nkvh, self.dh, half)
        if ctx.decode and self._decode_kernel(ctx, qkv, o, cache, table, nt, sfx):
            matmul_nt(o, self.weights["wo"], out)
            return
        if self.tc_tile and nt >= 2 * ctx.B and USE_TCGEN05:
            # prompts: S and O in tensor memory, K and V pages by TMA
            tiles = ctx.tiles(self.tc_tile)
            if lib.try_call("tb_attention_tc_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos),
                            lib.ptr(table), tiles.count, nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh,
                            self.dh, cache.k.shape[0], self.scale):
                matmul_nt(o, self.weights["wo"], out)
                return
        if self.prompt_tile and nt >= 2 * ctx.B:
            tiles = ctx.tiles(self.prompt_tile)
            if lib.try_call("tb_attention_prefill_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos),
                            lib.ptr(table), tiles.count, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                            self.scale):
                matmul_nt(o, self.weights["wo"], out)
                return
        tiles = ctx.tiles(self.general_tile)
        splits = ctx.attention_splits(tiles.count, self.nh, self.nkvh)
        partial = None
        if splits > 1:
            partial = ctx.scratch("attn.partial", (nt, self.nh, splits, self.dh + 2), torch.float32)
        lib.call("tb_attention_" + sfx, lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                 lib.ptr(tiles.seq), lib.ptr(tiles.t0), lib.ptr(tiles.nq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                 lib.ptr(partial), tiles.count, nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                 splits, self.scale)
        matmul_nt(o, self.weights["wo"], out)

    def _ring(self) -> bool:
        """Whether decoding runs the kernel with a ring of cache pages (TMA, tensor cores)."""
        return USE_DECODE_RING and self.dtype == torch.bfloat16 and self.dh in (64, 128, 192, 256)

    def _decode_plan(self, ctx, nt, ring):
        """Slices of the keys, and the scratch they need: (splits, partial results, counters of finished slices)."""
        group = self.nh // self.nkvh
        gc = 16 if ring else 1 if group == 1 else 2 if group == 2 else 4       # query heads of a group per block
        blocks = nt * self.nkvh * ((group + gc - 1) // gc)
        # Slices of the keys so that the blocks fill the GPU: as many blocks as are resident at once for the kernel
        # that keeps a ring of pages in shared memory (two per SM: measured best in the step at batch 1 to 16, also with
        # lengths that differ 16-fold; alone, the kernel would rather have one per SM), eight times the SMs for the register-staged one.  A function of the batch's shape
        # alone, since a captured graph keeps it for as long as the sequences grow (the kernels cut short sequences
        # into fewer slices by themselves).
        splits = int(max(1, min(32, ((RING_BLOCKS_PER_SM if ring else 8) * ctx.engine.sm_count) // blocks)))
        partial = done = None
        if splits > 1:
            partial = ctx.scratch("attn.partial", (nt, self.nh, splits, self.dh + 2), torch.float32)
            if ring:    # the block that finishes a head group's last slice merges them
                done = ctx.scratch("attn.done", (nt * self.nh,), torch.int32, zero=True)
        return splits, partial, done

    def _decode_fused(self, ctx, qkv, o, cache, table, nt, cos, sin, half) -> bool:
        """One token per sequence, straight from the q-k-v product: the ring kernel also rotates the queries and the
        new key and writes key and value into the cache.  False (and nothing done) if it refuses."""
        if not (self._ring() and FUSE_DECODE_ROPE):
            return False
        splits, partial, done = self._decode_plan(ctx, nt, True)
        return lib.try_call("tb_attention_decode_rope_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table), lib.ptr(partial), lib.ptr(done),
                            lib.ptr(cos), lib.ptr(sin), nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh,
                            splits, cache.k.shape[0], half, 1 if cache.writable else 0, self.scale)

    def _decode_kernel(self, ctx, qkv, o, cache, table, nt, sfx) -> bool:
        """One token per sequence, queries rotated and the cache written: the kernels that stream the cache.  False if
        they refuse the head size."""
        ring = self._ring()
        splits, partial, done = self._decode_plan(ctx, nt, ring)
        if ring:
            if lib.try_call("tb_attention_decode_mma_bf16", lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k),
                            lib.ptr(cache.v), lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table),
                            lib.ptr(partial), lib.ptr(done), nt, ctx.max_pages, self.qkv_width, self.nh, self.nkvh,
                            self.dh, splits, cache.k.shape[0], self.scale):
                return True
        return lib.try_call("tb_attention_decode_" + sfx, lib.ptr(qkv), lib.ptr(o), lib.ptr(cache.k), lib.ptr(cache.v),
                            lib.ptr(ctx.tok_seq), lib.ptr(ctx.tok_pos), lib.ptr(table), lib.ptr(partial), nt,
                            ctx.max_pages, self.qkv_width, self.nh, self.nkvh, self.dh, splits, self.scale)
