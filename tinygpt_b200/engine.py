"""Host-side mirror of tinygpt::GPTModel / GPTEngine for the greedy decode path, over the C-ABI engine.

  DecodeEngine.forward(ids)      ↔ GPTModel::forward → model()(inputIds)            [ref: src/model/GPTModel.h:86]
  DecodeEngine.reset_cache()     ↔ GPTModel::resetCache                             [ref: src/model/GPTModel.h:91-94]
  DecodeEngine.gen_next_token()  ↔ GPTEngine::genNextToken (greedy sampler)         [ref: src/engine/GPTEngine.cpp:94-99]
  DecodeEngine.generate_sync()   ↔ GPTEngine::generateSync, batch 1, greedy         [ref: src/engine/GPTEngine.cpp:154-174]
  DecodeEngine.generate_async()  ↔ GPTEngine::generateAsync + AsyncTokenPipeline    [ref: src/engine/GPTEngine.cpp:17-35,180-232]

torch is used for device memory, pinned host buffers and the current stream only.
"""
from __future__ import annotations

import ctypes as C
import time
from typing import Callable, Dict, Iterable, List, Optional, Tuple

import torch

from . import models
from ._lib import (AttnDesc, AttnPrepDesc, B200Error, DeltaDesc, GatedDeltaDesc, LatentDesc, LayerWeights, MambaDesc, MlstmDesc, ModelDesc,
                   MoeDesc, StackDesc, StackLayer, WeightTable, check, lib, require_device)


def align_prompts(token_lists, context_size: int, pad_token: int):
    """GPTEngine::encodeTexts' alignment of a ragged batch [ref: src/engine/GPTEngine.cpp:101-141]: the common length is
    min(longest prompt, context size); longer prompts keep their LAST tokens, shorter ones are padded on the LEFT with
    `pad_token` (the tokenizer's pad id, else eos, else 0 — the caller resolves that).  → (ids int64 [B, S], mask bool
    [B, S] with False on the pads; the reference builds the mask and then ignores it, and so does the engine)."""
    if len(token_lists) == 0:
        raise B200Error("align_prompts: empty batch")
    S = min(max(len(t) for t in token_lists), int(context_size))
    ids = torch.full((len(token_lists), S), int(pad_token), dtype=torch.int64)
    mask = torch.zeros((len(token_lists), S), dtype=torch.bool)
    for i, t in enumerate(token_lists):
        t = list(t)[-S:] if S > 0 else []
        if t:
            ids[i, S - len(t):] = torch.tensor(t, dtype=torch.int64)
            mask[i, S - len(t):] = True
    return ids, mask


class SequenceSlots:
    """Host-side owner of an engine's sequence slots: a request name gets the lowest free slot when it first appears
    and gives it back when it ends; a freed slot is handed out again (its cache rows are simply overwritten)."""

    def __init__(self, n_slots: int):
        self.n_slots = int(n_slots)
        self._free = list(range(self.n_slots))
        self._of: Dict[object, int] = {}

    def __contains__(self, name) -> bool:
        return name in self._of

    def __len__(self) -> int:
        return len(self._of)

    def slot(self, name) -> int:
        return self._of[name]

    def acquire(self, name) -> int:
        if name in self._of:
            return self._of[name]
        if not self._free:
            raise B200Error(f"no free sequence slot for {name!r}: all {self.n_slots} are taken")
        self._free.sort()
        s = self._free.pop(0)
        self._of[name] = s
        return s

    def release(self, name) -> int:
        s = self._of.pop(name)
        self._free.append(s)
        return s


class DecodeEngine:
    """Whole-token engine for ONE sequence (batch 1) on the current CUDA device.

    `weights` is a dict with the reference's merged layout (models.synth_weights) already on the device; the engine
    borrows the tensors (keeps references) and owns only its KV cache + workspace."""

    def __init__(self, spec: models.ModelSpec, weights: Dict[str, torch.Tensor], rope_table: Optional[torch.Tensor] = None):
        require_device()
        self.spec = spec
        self.is_stack = isinstance(spec, models.StackSpec)
        if self.is_stack:
            self._init_stack(spec, weights)
            return
        dev = weights["model.embed_tokens.weight"].device
        if dev.type != "cuda":
            raise B200Error("DecodeEngine: weights must be on a CUDA device (no CPU path)")
        self.device = dev
        self._w = weights  # keep alive
        if rope_table is None:
            # built on the device by the same fp32 powf/cosf/sinf kernels as the reference's op::ropeInit, so the table
            # is the one RoPE::cache() holds in a TinyGPT process (models.rope_table is the host/numpy restatement the
            # CPU oracle uses; libm and CUDA differ in the last bit of a few entries)
            from . import ops
            with torch.cuda.device(dev):
                rope_table = ops.rope_init(spec.head_dim, spec.max_ctx, spec.rope_theta, spec.rope_scaling, device=dev)
        self._rope = rope_table.to(dev).contiguous()
        self.local_vocab = spec.vocab
        desc, table = self._describe(spec, weights, rank=0, world=1, shard_attn=True)
        h = C.c_void_p()
        with torch.cuda.device(dev):
            check(lib().b200_engine_create(C.byref(desc), C.byref(table), C.byref(h)), "b200_engine_create")
        self._h = h

    def _describe(self, spec, weights, rank: int, world: int, shard_attn: bool):
        """ModelDesc + WeightTable over `weights` (merged layout; for TP the tensors are this rank's shards)."""
        L = spec.layers
        arr = (LayerWeights * L)()
        for l in range(L):
            p = f"model.layers.{l}."
            g = lambda k: self._ptr(weights.get(p + k))
            arr[l] = LayerWeights(g("input_layernorm.weight"), g("self_attn.qkv_proj.weight"),
                                  g("self_attn.qkv_proj.bias"), g("self_attn.q_norm.weight"),
                                  g("self_attn.k_norm.weight"), g("self_attn.o_proj.weight"),
                                  g("post_attention_layernorm.weight"), g("mlp.gate_up_proj.weight"),
                                  g("mlp.down_proj.weight"))
        head = weights.get("lm_head.weight")
        if head is None:
            head = weights["model.embed_tokens.weight"]
        self._layers = arr
        table = WeightTable(self._ptr(weights["model.embed_tokens.weight"]), self._ptr(weights["model.norm.weight"]),
                            self._ptr(head), self._rope.data_ptr(), arr)
        desc = ModelDesc(spec.hidden, L, spec.q_heads, spec.kv_heads, spec.head_dim, spec.intermediate, spec.vocab,
                         spec.max_ctx, spec.rms_eps, int(spec.qkv_bias), int(spec.qk_norm), rank, world,
                         int(shard_attn))
        return desc, table

    def _init_stack(self, spec: "models.StackSpec", weights: Dict[str, torch.Tensor]) -> None:
        """Layer-stack model (models.StackSpec; weights from models.pack_stack_weights / loader.load_stack_checkpoint):
        the description travels as data through b200_engine_create_stack."""
        dev = weights["embed"].device
        if dev.type != "cuda":
            raise B200Error("DecodeEngine: weights must be on a CUDA device (no CPU path)")
        self.device = dev
        self._w = weights
        self._rope = None
        self.local_vocab = spec.vocab
        mdt = weights["embed"].dtype
        if mdt not in (torch.bfloat16, torch.float32):
            raise B200Error("DecodeEngine: stack matrices must be bf16 or fp32")
        self.dtype = mdt

        def ptr(name, dt):
            t = weights.get(name)
            if t is None:
                return None
            if t.dtype != dt or not t.is_contiguous() or t.device != dev:
                raise B200Error(f"DecodeEngine: {name} must be a contiguous {dt} tensor on {dev}")
            return t.data_ptr()

        acts = {"gelu_tanh": 0, "silu": 1, "gelu_erf": 2, "relu2": 3, "tanh": 4}
        arr = (StackLayer * len(spec.layers))()
        sandwich = spec.block != "parallel"   # a descriptor per sublayer: sandwich and post-norm blocks
        self._rot_tables = {}
        self._mix_seen = False
        for i, L in enumerate(spec.layers if sandwich else ()):
            arr[i] = (self._postnorm_layer if spec.block == "postnorm" else self._sandwich_layer)(spec, i, L, ptr, mdt, acts)
        for i, L in enumerate(() if sandwich else spec.layers):
            a, lay, p = L.attn, spec.layout(i), f"l{i}."
            side = spec.side_dim > 0
            arr[i] = StackLayer(AttnDesc(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first,
                                         int(a.out_gate)),
                                L.ff, acts[L.ff_act], lay.off_q, lay.off_k, lay.off_v, lay.off_g, lay.off_gate,
                                lay.off_up, lay.n_in, lay.off_act, lay.k_out,
                                ptr(p + "norm", torch.float32), ptr(p + "w_in", mdt), ptr(p + "b_in", torch.float32),
                                ptr(p + "w_out", mdt), i * spec.side_dim,
                                ptr(p + "side_gate", mdt) if side else None, ptr(p + "side_proj", mdt) if side else None,
                                ptr(p + "side_norm", torch.float32) if side else None)
        runs = spec.runs()
        run_layer = (C.c_int32 * len(runs))(*[r[0] for r in runs])
        run_mix = (C.c_int32 * len(runs))(*[int(r[1]) for r in runs])
        desc = StackDesc(1 if mdt == torch.float32 else 0, {"parallel": 0, "sandwich": 1, "postnorm": 2}[spec.block], spec.width, spec.vocab, len(spec.layers), len(runs),
                         run_layer, run_mix, spec.embed_scale, spec.residual_mult, spec.norm_eps, spec.norm_offset,
                         spec.side_dim, spec.side_dim * len(spec.layers), spec.max_ctx, spec.max_slots,
                         ptr("embed", mdt), ptr("mix_in", mdt), ptr("side_table", mdt), ptr("final_norm", torch.float32),
                         ptr("head", mdt), arr, {"rms": 0, "layer": 1}[spec.norm_kind], spec.logit_softcap)
        h = C.c_void_p()
        with torch.cuda.device(dev):
            check(lib().b200_engine_create_stack(C.byref(desc), C.byref(h)), "b200_engine_create_stack")
        self._h = h
        self.slots = SequenceSlots(spec.max_slots)

    def _sandwich_layer(self, spec, i, L, ptr, mdt, acts) -> StackLayer:
        """Descriptor of layer i of a sandwich-block model (latent attention, mLSTM, prepared attention or gated delta rule
        mixer; dense or routed feed-forward); the rotation tables are built here, for the engine's context length."""
        lay, p = spec.mix_layout(i), f"l{i}."
        f32 = torch.float32
        lat, rec, moe, prep, gdelta = LatentDesc(), MlstmDesc(), MoeDesc(), AttnPrepDesc(), GatedDeltaDesc()
        kv_share = 0

        def table(rot):
            tab = self._rot_tables.get(rot)
            if tab is None and rot is not None and rot.dims > 0:
                tab = self._rot_tables[rot] = rot.table(spec.max_ctx).contiguous().to(self.device)
            return tab

        if L.mixer == "latent_attention":
            a = L.latent
            attn = AttnDesc(a.heads, 1, a.dim, a.vdim, a.scale, a.window, 0, 0)
            tab = table(a.rot)
            lat = LatentDesc(a.kv_rank, a.rot_dim, a.rot.dims, ptr(p + "c_norm", f32), ptr(p + "uk_t", mdt), ptr(p + "uk", mdt),
                             ptr(p + "uv", mdt),
                             tab.data_ptr() if tab is not None else None, int(a.rot_layout == "half"), a.q_rank,
                             ptr(p + "q_norm", f32) if a.q_rank > 0 else None, ptr(p + "uq", mdt) if a.q_rank > 0 else None,
                             int(a.out_gate))
            mixer = 1
        elif L.mixer == "attention":
            a, q = L.attn, L.prep or models.AttnPrepSpec()
            attn = AttnDesc(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first, int(a.out_gate), int(a.sink))
            tab = table(q.rot)
            if q.v_mix:
                raise B200Error(f"DecodeEngine: layer {i}: the value mix-in is built for post-norm blocks")
            prep = AttnPrepDesc(int(q.qk_norm), q.rot.dims if q.rot is not None else 0, int(q.v_norm), 0,
                                ptr(p + "q_norm", f32) if q.qk_norm else None, ptr(p + "k_norm", f32) if q.qk_norm else None,
                                tab.data_ptr() if tab is not None else None, None, int(q.rot_interleaved))
            kv_share = 0 if L.kv_from is None else L.kv_from + 1
            mixer = 0
        elif L.mixer == "gated_delta":
            a = L.gdelta
            attn = AttnDesc(a.heads, a.kv_heads, a.dim, a.vdim, 1.0, 0, 0, 0)
            gdelta = GatedDeltaDesc(a.conv, a.unit_eps, ptr(p + "conv_w", f32), ptr(p + "A_log", f32), ptr(p + "dt_bias", f32),
                                    ptr(p + "head_norm", f32))
            mixer = 5
        else:
            a = L.mlstm
            attn = AttnDesc(a.heads, a.heads, a.dim, a.vdim, 1.0, 0, 0, 0)
            rec = MlstmDesc(a.gate_cap, ptr(p + "head_norm", f32))
            mixer = 2
        has_ff = L.ff_kind == "moe" or L.ff > 0
        if L.ff_kind == "moe":
            m = L.moe
            moe = MoeDesc(m.experts, m.top, m.expert_ff, m.shared_ff, m.limit, m.shared_limit, ptr(p + "router", mdt),
                          ptr(p + "w_exp_in", mdt), ptr(p + "w_exp_out", mdt))
        return StackLayer(attn, L.ff, acts[L.ff_act], lay.off_q, lay.off_k, lay.off_v, lay.off_g, lay.off_gate, lay.off_up, lay.n_in,
                          0, lay.k_out, ptr(p + "norm", f32), ptr(p + "w_in", mdt), ptr(p + "b_in", f32), ptr(p + "w_out", mdt),
                          0, None, None, None, mixer, 2 if L.ff_kind == "moe" else 1, ptr(p + "post_norm", f32),
                          ptr(p + "ff_norm", f32) if has_ff else None, ptr(p + "ff_post_norm", f32) if has_ff else None,
                          ptr(p + "w_ff_in", mdt), ptr(p + "w_ff_out", mdt), lat, rec, moe, prep, DeltaDesc(), MambaDesc(), gdelta,
                          ptr(p + "b_out", f32), kv_share)

    def _postnorm_layer(self, spec, i, L, ptr, mdt, acts) -> StackLayer:
        """Descriptor of layer i of a post-norm-block model (prepared attention, generalized delta rule or Mamba-2 mixer;
        routed feed-forward or none); rotation tables are built here, for the engine's context length."""
        lay, p = spec.mix_layout(i), f"l{i}."
        f32 = torch.float32
        moe, prep, delta, mamba = MoeDesc(), AttnPrepDesc(), DeltaDesc(), MambaDesc()
        if L.mixer == "attention":
            a, q = L.attn, L.prep
            attn = AttnDesc(a.heads, a.kv_heads, a.dim, a.vdim, a.scale, a.window, a.keep_first, int(a.out_gate))
            tab = None
            if q.rot is not None:
                tab = self._rot_tables.get(q.rot)
                if tab is None:
                    tab = self._rot_tables[q.rot] = q.rot.table(spec.max_ctx).contiguous().to(self.device)
            v_mix = 0
            if q.v_mix:   # the first such layer keeps its values, the later ones mix them in
                v_mix = 2 if self._mix_seen else 1
                self._mix_seen = True
            prep = AttnPrepDesc(int(q.qk_norm), q.rot.dims if q.rot is not None else 0, int(q.v_norm), v_mix,
                                ptr(p + "q_norm", f32) if q.qk_norm else None, ptr(p + "k_norm", f32) if q.qk_norm else None,
                                tab.data_ptr() if tab is not None else None, ptr(p + "vmix", f32) if v_mix == 2 else None)
            mixer = 0
        elif L.mixer == "general_delta":
            a = L.delta
            attn = AttnDesc(a.heads, a.heads, a.dim, a.dim, 1.0, 0, 0, 0)
            delta = DeltaDesc(a.rank, a.decay_scale, a.unit_eps, ptr(p + "w2", mdt), ptr(p + "w0", f32), ptr(p + "head_norm", f32))
            mixer = 3
        elif L.mixer == "mamba2":
            a = L.mamba
            attn = AttnDesc(a.heads, a.groups, a.state, a.vdim, 1.0, 0, 0, 0)
            mamba = MambaDesc(a.state, a.groups, a.conv, a.norm_groups, ptr(p + "conv_w", f32), ptr(p + "conv_b", f32),
                              ptr(p + "dt_bias", f32), ptr(p + "A_log", f32), ptr(p + "D", f32), ptr(p + "mix_norm", f32))
            mixer = 4
        else:
            raise B200Error(f"DecodeEngine: layer {i}: mixer {L.mixer!r} is not built for post-norm blocks")
        has_ff = L.ff_kind == "moe" or L.ff > 0
        if L.ff_kind == "moe":
            m = L.moe
            moe = MoeDesc(m.experts, m.top, m.expert_ff, m.shared_ff, m.limit, m.shared_limit, ptr(p + "router", mdt),
                          ptr(p + "w_exp_in", mdt), ptr(p + "w_exp_out", mdt), {"sigmoid": 0, "softmax": 1}[m.router],
                          int(m.weight_output), 0 if m.act == "glu_clamp" else acts[m.act], int(m.shared_plain), m.route_scale)
        return StackLayer(attn, L.ff, acts[L.ff_act], lay.off_q, lay.off_k, lay.off_v, lay.off_g, lay.off_gate, lay.off_up,
                          lay.n_in, 0, lay.k_out, None, ptr(p + "w_in", mdt),
                          ptr(p + "b_in", f32) if L.mixer == "general_delta" else None,   # the only in-projection with a bias
                          ptr(p + "w_out", mdt),
                          0, None, None, None, mixer, 2 if L.ff_kind == "moe" else 1, ptr(p + "post_norm", f32),
                          None, ptr(p + "ff_post_norm", f32) if has_ff else None,
                          ptr(p + "w_ff_in", mdt), ptr(p + "w_ff_out", mdt), LatentDesc(), MlstmDesc(), moe, prep, delta, mamba)

    # --------------------------------------------------------------------------------- ragged steps (stack engines)
    def step(self, entries, greedy: bool = False) -> torch.Tensor:
        """One ragged step.  `entries`: list of (slot, tokens, want) — `tokens` the sequence's next token ids, `want`
        the places among them whose logits are returned.  → fp32 [Σ len(want), vocab] on the device, in the order of
        the entries and of their `want`.  greedy: the last token of every entry also chooses that slot's next token, and
        the entries become the batch `decode` continues."""
        if not self.is_stack:
            raise B200Error("DecodeEngine.step: ragged steps need a layer-stack model")
        n = len(entries)
        slots = (C.c_int32 * n)(*[int(e[0]) for e in entries])
        counts = (C.c_int32 * n)(*[len(e[1]) for e in entries])
        flat = [int(t) for e in entries for t in e[1]]
        ids = (C.c_int64 * max(1, len(flat)))(*flat)
        want, base = [], 0
        for e in entries:
            for k in e[2]:
                if not 0 <= int(k) < len(e[1]):
                    raise B200Error(f"DecodeEngine.step: wanted place {k} outside the entry's {len(e[1])} tokens")
                want.append(base + int(k))
            base += len(e[1])
        wa = (C.c_int32 * max(1, len(want)))(*want)
        out = torch.empty(len(want), self.spec.vocab, dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            check(lib().b200_engine_step(self._h, n, slots, counts, ids, len(want), wa,
                                         out.data_ptr() if want else None, int(greedy), self._stream()), "b200_engine_step")
        if greedy:
            self._batch = n
        return out

    def release(self, slot: int) -> None:
        """The sequence in `slot` is over: position back to 0, the slot leaves the active batch."""
        check(lib().b200_engine_slot_reset(self._h, int(slot), self._stream()), "b200_engine_slot_reset")

    def slot_position(self, slot: int) -> int:
        return int(lib().b200_engine_slot_position(self._h, int(slot)))

    def generate_ragged(self, prompts, max_new_tokens: int) -> List[List[int]]:
        """Greedy generation for prompts of unequal length WITHOUT padding (stack engines): one ragged prefill step,
        then max_new_tokens - 1 batched decode steps on the device; sequence i lives in slot i."""
        if max_new_tokens < 1 or not prompts or len(prompts) > self.spec.max_slots:
            raise B200Error("generate_ragged: 1 … max_slots prompts and at least one new token")
        self.reset_cache()
        self.step([(i, list(p), []) for i, p in enumerate(prompts)], greedy=True)
        first = torch.empty(len(prompts), 1, dtype=torch.int64, device=self.device)
        check(lib().b200_engine_last_token(self._h, first.data_ptr(), self._stream()), "b200_engine_last_token")
        rest = self.decode(max_new_tokens - 1).view(max_new_tokens - 1, -1).t()
        return torch.cat([first, rest], dim=1).cpu().tolist()

    @staticmethod
    def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
        if t is None:
            return None
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise B200Error("DecodeEngine: weights must be contiguous bf16 tensors")
        return t.data_ptr()

    def close(self) -> None:
        if getattr(self, "_h", None) is not None and self._h:
            lib().b200_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------------------------------------ state
    def _stream(self) -> int:
        return torch.cuda.current_stream(self.device).cuda_stream

    @property
    def rope_table(self) -> torch.Tensor:
        """fp32 [max_ctx, head_dim, 2] cos/sin table the engine rotates with."""
        return self._rope

    @property
    def position(self) -> int:
        return int(lib().b200_engine_position(self._h))

    @property
    def launches_per_token(self) -> int:
        return int(lib().b200_engine_launches_per_token(self._h))

    @property
    def options(self) -> dict:
        """Code paths this engine was built with (b200_engine_options)."""
        o = int(lib().b200_engine_options(self._h))
        return {"cuda_graph": bool(o & 1), "pdl": bool(o & 2), "gemm_prefill": bool(o & 8)}

    def bytes_per_token(self, ctx: int) -> int:
        return int(lib().b200_engine_bytes_per_token(self._h, ctx))

    def reset_cache(self) -> None:
        check(lib().b200_engine_reset(self._h, self._stream()), "b200_engine_reset")

    def seek(self, position: int) -> None:
        """Rewind to `position` inside the cached prefix (rows below it stay valid)."""
        check(lib().b200_engine_seek(self._h, int(position), self._stream()), "b200_engine_seek")

    # ---------------------------------------------------------------------------------------------- forward
    def forward(self, ids: torch.Tensor, all_positions: bool = False) -> torch.Tensor:
        """ids [1, S] int64 on the device → logits [1, S, V] (all_positions) or [1, 1, V] (last position) bf16.
        (Tensor-parallel engines return this rank's vocabulary shard, V / world columns.)"""
        max_b = self.spec.max_slots if self.is_stack else 8
        if ids.dim() != 2 or not 1 <= ids.shape[0] <= max_b:
            raise B200Error(f"DecodeEngine.forward: ids must be [B, S] with 1 ≤ B ≤ {max_b} (sequences at the same position)")
        if ids.dtype != torch.int64 or not ids.is_cuda:
            raise B200Error("DecodeEngine.forward: ids must be int64 on the device (reference: FuncNNLayer.h:205)")
        ids = ids.contiguous()
        B, S = ids.shape
        rows = S if all_positions else 1
        logits = torch.empty(B, rows, self.local_vocab, dtype=torch.bfloat16, device=self.device)
        check(lib().b200_engine_forward(self._h, ids.data_ptr(), B, S, logits.data_ptr(), int(all_positions),
                                        self._stream()), "b200_engine_forward")
        self._batch = B
        return logits

    def gen_next_token(self, ids: torch.Tensor) -> torch.Tensor:
        """genNextToken: forward → last position → greedy argmax (device tensor [B, 1] int64)."""
        B = ids.shape[0]
        check(lib().b200_engine_forward(self._h, ids.contiguous().data_ptr(), B, ids.shape[1], None, 0, self._stream()),
              "b200_engine_forward")
        self._batch = B
        out = torch.empty(B, 1, dtype=torch.int64, device=self.device)
        check(lib().b200_engine_last_token(self._h, out.data_ptr(), self._stream()), "b200_engine_last_token")
        return out

    def decode(self, n_steps: int) -> torch.Tensor:
        """n greedy steps on the device, each consuming the previous step's token → int64 [n] device tensor (after a
        batched forward with B > 1 sequences: [n, B])."""
        B = getattr(self, "_batch", 1)
        out = torch.empty((n_steps, B) if B > 1 else (n_steps,), dtype=torch.int64, device=self.device)
        check(lib().b200_engine_decode(self._h, n_steps, out.data_ptr(), self._stream()), "b200_engine_decode")
        return out

    def generate_sync_batch(self, prompts, max_new_tokens: int, pad_token: int = 0) -> torch.Tensor:
        """GPTEngine::generateSync for a batch of prompts with HOST buffers [ref: src/engine/GPTEngine.cpp:154-174]: one
        weight pass per step for the whole batch.  `prompts`: [B, S] ids, or a list of ragged id lists that is aligned
        the reference's way first (`align_prompts`: left padding with `pad_token`, truncation to the context; like the
        reference, the pad positions are attended — its mask is a TODO, GPTEngine.cpp:95).  → CPU int64 [B, new]."""
        if isinstance(prompts, (list, tuple)) and len(prompts) and not torch.is_tensor(prompts[0]) \
                and len({len(p) for p in prompts}) > 1:
            if self.is_stack:   # slots have their own positions: no padding, nothing attends a pad
                return torch.tensor(self.generate_ragged(prompts, max_new_tokens), dtype=torch.int64)
            prompts, _ = align_prompts(prompts, self.spec.max_ctx, pad_token)
        prompts = torch.as_tensor(prompts, dtype=torch.int64)
        if prompts.dim() != 2 or prompts.shape[0] < 1:
            raise B200Error("generate_sync_batch: prompts must be [B, S]")
        ids = prompts.pin_memory().to(self.device, non_blocking=True)
        self.reset_cache()
        first = self.gen_next_token(ids)                       # [B, 1]
        rest = self.decode(max_new_tokens - 1)                 # [n-1, B] (or [n-1] for B = 1)
        rest = rest.view(max_new_tokens - 1, -1).t()
        toks = torch.cat([first, rest], dim=1).cpu()
        return toks

    # ------------------------------------------------------------------------------------------ generateSync
    def generate_sync(self, prompt_ids: List[int] | torch.Tensor, max_new_tokens: int,
                      pinned_in: Optional[torch.Tensor] = None, pinned_out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """GPTEngine::generateSync for one sequence with HOST buffers: reset cache, H2D copy of the prompt ids,
        prefill, (max_new_tokens - 1) decode steps, ONE D2H copy of the generated ids (like the reference, no
        per-step host synchronisation).  Returns a CPU int64 tensor [max_new_tokens]."""
        if max_new_tokens < 1:
            raise B200Error("generate_sync: max_new_tokens must be >= 1")
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64).view(1, -1)
        if prompt.numel() == 0:
            raise B200Error("generate_sync: empty prompt")
        if pinned_in is None:
            pinned_in = torch.empty(prompt.shape, dtype=torch.int64).pin_memory()
        pinned_in.view(-1)[: prompt.numel()].copy_(prompt.view(-1))
        ids_dev = pinned_in.view(-1)[: prompt.numel()].to(self.device, non_blocking=True).view(1, -1)
        self.reset_cache()
        first = self.gen_next_token(ids_dev)
        rest = self.decode(max_new_tokens - 1)
        toks = torch.cat([first.view(-1), rest])
        if pinned_out is None:
            pinned_out = torch.empty(max_new_tokens, dtype=torch.int64).pin_memory()
        pinned_out[:max_new_tokens].copy_(toks, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        return pinned_out[:max_new_tokens].clone()

    # ------------------------------------------------------------------------------------------------ sampler
    def set_sampler(self, temperature: float = 0.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
                    seed: int = 0) -> None:
        """SamplerConfig of the reference's generate loop (src/engine/Sampler.h:13-22).  Any knob set ⇒ every token is
        drawn by the device sampler with u = philox_uniform(seed, tokens generated so far); all off ⇒ greedy."""
        check(lib().b200_engine_set_sampler(self._h, float(temperature), int(top_k), float(top_p), float(min_p),
                                            int(seed) & 0xFFFFFFFFFFFFFFFF, self._stream()), "b200_engine_set_sampler")

    @staticmethod
    def philox_uniform(seed: int, n: int) -> float:
        """The uniform number the engine's sampler uses for its n-th generated token (n counts from 0): Philox4x32-10,
        counter {n lo, n hi, 0, 0}, key = seed; u = ((x0 >> 8) + 0.5)·2^-24.  Host mirror of sampling.cu."""
        M = 0xFFFFFFFF
        c = [n & M, (n >> 32) & M, 0, 0]
        k = [seed & M, (seed >> 32) & M]
        for _ in range(10):
            p0, p1 = 0xD2511F53 * c[0], 0xCD9E8D57 * c[2]
            c = [((p1 >> 32) ^ c[1] ^ k[0]) & M, p1 & M, ((p0 >> 32) ^ c[3] ^ k[1]) & M, p0 & M]
            k = [(k[0] + 0x9E3779B9) & M, (k[1] + 0xBB67AE85) & M]
        return ((c[0] >> 8) + 0.5) / 16777216.0

    # ----------------------------------------------------------------------------------------- generateAsync
    def set_mailbox(self, capacity: int = 64) -> torch.Tensor:
        """Attach a token mailbox: a zeroed ring of `capacity` 8-byte words in pinned host memory that the argmax kernel
        posts {sequence tag, token} into (b200_engine_set_mailbox).  Returns the ring (int64 view of the words)."""
        ring = torch.zeros(capacity, dtype=torch.int64).pin_memory()
        check(lib().b200_engine_set_mailbox(self._h, ring.data_ptr(), capacity, self._stream()),
              "b200_engine_set_mailbox")
        self._ring, self._ring_np = ring, ring.numpy()  # numpy view: every element read is a fresh load
        return ring

    def clear_mailbox(self) -> None:
        check(lib().b200_engine_set_mailbox(self._h, None, 0, self._stream()), "b200_engine_set_mailbox")
        self._ring = self._ring_np = None

    def _fetch_token(self, n: int, timeout_s: float = 30.0) -> int:
        """Token number n (1-based count of tokens this engine generated) from the mailbox; spins on host memory."""
        cap = self._ring_np.shape[0]
        tag = n & 0xFFFFFFFF
        t0 = None
        while True:
            word = int(self._ring_np[(n - 1) % cap]) & 0xFFFFFFFFFFFFFFFF
            if (word >> 32) == tag:
                return word & 0xFFFFFFFF
            if t0 is None:
                t0 = time.perf_counter()
            elif time.perf_counter() - t0 > timeout_s:
                raise B200Error(f"generate_async: token {n} did not arrive within {timeout_s} s")

    def generate_async(self, prompt_ids, max_new_tokens: int, callback: Optional[Callable[[int], bool]] = None,
                       eos_ids: Iterable[int] = (), lookahead: int = 4) -> Tuple[List[int], str]:
        """GPTEngine::generateAsync for one sequence, greedy: tokens are handed to `callback(token_id) -> keep_going`
        as they are produced while the engine already runs up to `lookahead` steps ahead; no stream synchronisation or
        memcpy per token (the reference blocks on Tensor::item() for each one).  Stops at an EOS id (not passed to the
        callback, like the reference), when the callback returns False, or after max_new_tokens.
        Returns (token ids handed out, finish reason 'stop' | 'length').  Afterwards the engine is positioned so that
        feeding the next input token continues the sequence (steps that ran ahead of the stop are rewound)."""
        if max_new_tokens < 1:
            raise B200Error("generate_async: max_new_tokens must be >= 1")
        if getattr(self, "_ring_np", None) is None:
            self.set_mailbox(max(64, 4 * lookahead))
        if lookahead < 1 or lookahead >= self._ring_np.shape[0]:
            raise B200Error("generate_async: lookahead must be in [1, mailbox capacity)")
        eos = set(int(t) for t in eos_ids)
        prompt = torch.as_tensor(prompt_ids, dtype=torch.int64).view(1, -1)
        if prompt.numel() == 0:
            raise B200Error("generate_async: empty prompt")
        S = prompt.shape[1]
        self.reset_cache()
        base = self._generated()                               # tokens generated before this call
        self._enqueue_prefill(prompt)
        launched, out, reason = 1, [], "length"
        while len(out) < max_new_tokens:
            while launched < max_new_tokens and launched - len(out) < lookahead:
                self._enqueue_step()
                launched += 1
            tok = self._fetch_token(base + len(out) + 1)
            if tok in eos:
                reason = "stop"
                break
            out.append(tok)
            if callback is not None and not callback(tok):
                reason = "stop"
                break
        self._drain()
        # position of the next input token = S + (tokens kept) - 1 … the last kept token has not been fed yet unless a
        # look-ahead step consumed it; rewinding there makes both cases equal
        keep = max(len(out), 1)
        if S + keep - 1 < self.position:
            self.seek(S + keep - 1)
        return out, reason

    # the four touch points of generate_async with the device (overridden by the host-logic test's fake engine)
    def _generated(self) -> int:
        return int(lib().b200_engine_generated(self._h))

    def _enqueue_prefill(self, prompt: torch.Tensor) -> None:
        ids_dev = prompt.pin_memory().to(self.device, non_blocking=True)
        check(lib().b200_engine_forward(self._h, ids_dev.data_ptr(), 1, prompt.shape[1], None, 0, self._stream()),
              "b200_engine_forward")

    def _enqueue_step(self) -> None:
        check(lib().b200_engine_decode(self._h, 1, None, self._stream()), "b200_engine_decode")

    def _drain(self) -> None:
        torch.cuda.current_stream(self.device).synchronize()
