"""Checkpoint loading: HF safetensors names -> model parameters, with format conversion.

Accepted weight formats (per tensor):
  * bf16 / fp16 / fp32
  * HF DeepSeek-V3 e4m3 + ``weight_scale_inv`` fp32 per 128x128 block (loaded as is)
  * compressed-tensors int8 w8a8: ``weight`` int8 [out,in] + ``weight_scale`` [out,1] (+ ``weight_offset``)
    as produced for the reference (omni/quantization/compressed_tensors/schemes/compressed_tensors_w8a8_int8.py:33-69,
    omni/quantization/compressed_tensors/compressed_tensors_moe.py:34-92); dequantised at load and re-quantised
    to block-scaled e4m3 when the target layer is quantised.
Stacked parameters: q_a_proj + kv_a_proj_with_mqa -> fused_qkv_a_proj, gate_proj + up_proj -> gate_up_proj,
q/k/v_proj -> qkv_proj, experts.{e}.{gate,up,down}_proj -> w13 / w2 slots chosen by the placement pattern
(omni/models/deepseek/deepseek_v3.py:800-895, omni/models/common/layers/moe/fused_moe/layer.py:410-532).
"""
from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Iterable, Optional

import torch

from ..ops import FP8
from ..ops.gemm import dequant_weight_ref, quant_weight_fp8_block_ref


def _to_float(w: torch.Tensor, scale: Optional[torch.Tensor], offset: Optional[torch.Tensor]) -> torch.Tensor:
    if w.dtype == FP8:
        return dequant_weight_ref(w, scale) if scale is not None else w.float()
    if w.dtype == torch.int8:
        f = w.float()
        if offset is not None:
            f = f - offset.float().view(-1, 1)
        return f * scale.float().view(-1, 1)
    return w.float()


class WeightLoader:
    def __init__(self, model, cfg, planner=None, mtp_layer: Optional[int] = None):
        self.model, self.cfg, self.planner, self.mtp_layer = model, cfg, planner, mtp_layer
        self.params = dict(model.named_parameters())
        self.loaded: set = set()
        self._pending: dict = {}     # base name -> {"weight":..., "scale":..., "offset":...}

    # -- write one logical weight (float or fp8+scale) into (a row slice of) a parameter
    def _store(self, pname: str, sname: Optional[str], w, scale, offset, rows=None, index=None):
        p = self.params[pname]
        tgt = p.data if index is None else p.data[index]
        slice_fn = getattr(p, "tp_slice_fn", None)
        if slice_fn is not None and rows is None and index is None:
            # tensor-parallel shard of a whole checkpoint tensor (merged projections are not sharded by this route)
            if p.dtype == FP8 and not (w.dtype == FP8 and scale is not None):
                w, scale = quant_weight_fp8_block_ref(_to_float(w, scale, offset).to(tgt.device))
                offset = None
            if p.dtype == FP8:
                scale = self.params[sname].tp_slice_fn(scale)
            elif scale is not None:
                w, scale, offset = _to_float(w, scale, offset), None, None
            w = slice_fn(w)
        r0, r1 = rows if rows is not None else (0, tgt.shape[0])
        if p.dtype == FP8:
            sp = self.params[sname]
            stgt = sp.data if index is None else sp.data[index]
            if w.dtype == FP8 and scale is not None:
                tgt[r0:r1].copy_(w)
                stgt[r0 // 128:(r1 + 127) // 128].copy_(scale)
            else:
                q, s = quant_weight_fp8_block_ref(_to_float(w, scale, offset).to(tgt.device))
                tgt[r0:r1].copy_(q)
                stgt[r0 // 128:(r1 + 127) // 128].copy_(s)
            self.loaded.add(sname)
        else:
            tgt[r0:r1].copy_(_to_float(w, scale, offset).to(p.dtype))
        self.loaded.add(pname)

    def _slot_for_expert(self, layer_idx: int, expert: int, moe):
        """Local slots that hold logical expert ``expert`` on this rank (placement pattern aware)."""
        if self.planner is not None:
            return self.planner.local_slots_of(moe.moe_index, expert)
        return moe.local_slots_of(expert)

    def _route(self, name: str, w, scale, offset):
        cfg = self.cfg
        m = re.match(r"model\.layers\.(\d+)\.(.*)", name)
        if self.mtp_layer is not None:
            # drafter: only layer `mtp_layer`; its sub-names map onto enorm / hnorm / eh_proj / shared_head / decoder
            if not m or int(m.group(1)) != self.mtp_layer:
                return
            rest = m.group(2)
            simple = {"enorm.weight": "enorm.weight", "hnorm.weight": "hnorm.weight", "eh_proj.weight": "eh_proj.weight",
                      "shared_head.norm.weight": "shared_head_norm.weight"}
            if rest in simple:
                return self._store(simple[rest], None, w, scale, offset)
            if rest.startswith(("embed_tokens", "shared_head.head")):
                return   # shared with the main model
            return self._route_layer("decoder.", self.model.decoder, int(m.group(1)), rest, w, scale, offset)
        if m:
            li = int(m.group(1))
            if li >= len(self.model.model.layers):
                return   # MTP layers are skipped by the main model
            return self._route_layer(f"model.layers.{li}.", self.model.model.layers[li], li, m.group(2), w, scale, offset)
        direct = {"model.embed_tokens.weight": "model.embed_tokens.weight", "model.norm.weight": "model.norm.weight",
                  "lm_head.weight": "lm_head.weight"}
        if name in direct and direct[name] in self.params:
            self._store(direct[name], None, w, scale, offset)

    def _route_layer(self, prefix, layer, li, rest, w, scale, offset):
        cfg = self.cfg
        P = lambda n: prefix + n   # noqa: E731
        if rest in ("input_layernorm.weight", "post_attention_layernorm.weight"):
            return self._store(P(rest), None, w, scale, offset)
        if rest.startswith("self_attn."):
            a = rest[len("self_attn."):]
            base = P("self_attn.")
            if cfg.use_mla:
                ql = cfg.q_lora_rank
                qdim = cfg.num_attention_heads * cfg.qk_head_dim
                table = {
                    "q_a_proj.weight": ("fused_qkv_a_proj", (0, ql)),
                    "kv_a_proj_with_mqa.weight": ("fused_qkv_a_proj", (ql, ql + cfg.kv_lora_rank + cfg.qk_rope_head_dim)) if ql
                    else ("fused_qkv_a_proj", (qdim, qdim + cfg.kv_lora_rank + cfg.qk_rope_head_dim)),
                    "q_proj.weight": ("fused_qkv_a_proj", (0, qdim)),
                    "q_b_proj.weight": ("q_b_proj", None), "kv_b_proj.weight": ("kv_b_proj", None),
                    "o_proj.weight": ("o_proj", None),
                }
                if a in ("q_a_layernorm.weight", "kv_a_layernorm.weight"):
                    return self._store(base + a, None, w, scale, offset)
            else:
                Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
                table = {
                    "q_proj.weight": ("qkv_proj", (0, Hq * D)), "k_proj.weight": ("qkv_proj", (Hq * D, (Hq + Hkv) * D)),
                    "v_proj.weight": ("qkv_proj", ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)), "o_proj.weight": ("o_proj", None),
                }
                if a in ("q_norm.weight", "k_norm.weight"):
                    return self._store(base + a, None, w, scale, offset)
                att = layer.self_attn
                if getattr(att, "tp_world", 1) > 1 and a[:2] in ("q_", "k_", "v_") and a[2:] in ("proj.weight", "proj.bias"):
                    # tensor-parallel attention: this rank's heads of the checkpoint tensor, into the local merged rows
                    (s0, s1), rows = att.tp_ckpt_rows(a[0])
                    if a.endswith("bias"):
                        self.params[base + "qkv_proj.bias"].data[rows[0]:rows[1]].copy_(w[s0:s1])
                        self.loaded.add(base + "qkv_proj.bias")
                        return
                    if w.dtype == FP8 and scale is not None and s0 % 128 == 0 and s1 % 128 == 0:
                        w, scale = w[s0:s1], scale[s0 // 128:s1 // 128]
                    else:
                        w, scale, offset = _to_float(w, scale, offset)[s0:s1], None, None
                    return self._store(base + "qkv_proj.weight", base + "qkv_proj.weight_scale", w, scale, offset, rows=rows)
                bias = {"q_proj.bias": (0, Hq * D), "k_proj.bias": (Hq * D, (Hq + Hkv) * D),
                        "v_proj.bias": ((Hq + Hkv) * D, (Hq + 2 * Hkv) * D)}
                if a in bias:
                    r0, r1 = bias[a]
                    self.params[base + "qkv_proj.bias"].data[r0:r1].copy_(w)
                    self.loaded.add(base + "qkv_proj.bias")
                    return
            if a in table:
                mod, rows = table[a]
                return self._store(base + mod + ".weight", base + mod + ".weight_scale", w, scale, offset, rows=rows)
            return
        if rest.startswith("mlp."):
            a = rest[len("mlp."):]
            base = P("mlp.")
            if not getattr(layer, "is_moe", False):
                I = cfg.intermediate_size
                table = {"gate_proj.weight": ("gate_up_proj", (0, I)), "up_proj.weight": ("gate_up_proj", (I, 2 * I)),
                         "down_proj.weight": ("down_proj", None)}
                if a in table:
                    mod, rows = table[a]
                    self._store(base + mod + ".weight", base + mod + ".weight_scale", w, scale, offset, rows=rows)
                return
            moe = layer.mlp
            if a == "gate.weight":
                return self._store(base + "gate.weight", None, w, scale, offset)
            if a == "gate.e_score_correction_bias":
                return self._store(base + "gate.e_score_correction_bias", None, w, scale, offset)
            ms = re.match(r"shared_experts?\.(gate_proj|up_proj|down_proj)\.weight", a)
            if ms and getattr(moe, "shared_ranks", 0):
                # dedicated shared-expert ranks: piece j of the shared expert (a block of its intermediate dimension) goes
                # to local slot j there; the other ranks hold nothing of it
                if moe.ep_rank >= moe.shared_ranks:
                    return
                I, which = cfg.moe_intermediate_size, ms.group(1)
                blk = w.dtype == FP8 and scale is not None and I % 128 == 0
                if not blk:
                    w, scale, offset = _to_float(w, scale, offset), None, None
                for j in range(moe.shared_pieces):
                    if which == "down_proj":
                        self._store(base + "w2", base + "w2_scale", w[:, j * I:(j + 1) * I],
                                    scale[:, j * I // 128:(j + 1) * I // 128] if blk else None, None, index=j)
                    else:
                        self._store(base + "w13", base + "w13_scale", w[j * I:(j + 1) * I],
                                    scale[j * I // 128:(j + 1) * I // 128] if blk else None, None,
                                    rows=(0, I) if which == "gate_proj" else (I, 2 * I), index=j)
                return
            if ms:
                I = cfg.moe_intermediate_size * cfg.n_shared_experts
                mod, rows = {"gate_proj": ("gate_up_proj", (0, I)), "up_proj": ("gate_up_proj", (I, 2 * I)),
                             "down_proj": ("down_proj", None)}[ms.group(1)]
                return self._store(base + f"shared_experts.{mod}.weight", base + f"shared_experts.{mod}.weight_scale",
                                   w, scale, offset, rows=rows)
            me = re.match(r"experts\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight", a)
            if me:
                e, which = int(me.group(1)), me.group(2)
                I = cfg.moe_intermediate_size
                for slot in self._slot_for_expert(li, e, moe):
                    if which == "down_proj":
                        self._store(base + "w2", base + "w2_scale", w, scale, offset, index=slot)
                    else:
                        rows = (0, I) if which == "gate_proj" else (I, 2 * I)
                        self._store(base + "w13", base + "w13_scale", w, scale, offset, rows=rows, index=slot)

    def load(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set:
        """Consume (name, tensor) pairs in any order; scale / offset tensors are paired with their weight."""
        for name, t in weights:
            mm = re.match(r"(.*)\.(weight_scale_inv|weight_scale|weight_offset|weight)$", name)
            if not mm or not (t.dtype in (FP8, torch.int8) or mm.group(2) != "weight" or (mm.group(1) + ".weight") in self._pending):
                # plain tensor (norms, biases, unquantised weights)
                if name.endswith(("weight_scale_inv", "weight_scale", "weight_offset")):
                    base = mm.group(1)
                    ent = self._pending.setdefault(base + ".weight", {})
                    ent["offset" if name.endswith("offset") else "scale"] = t
                    self._flush(base + ".weight")
                    continue
                self._route(name, t, None, None)
                continue
            base = mm.group(1) + ".weight"
            ent = self._pending.setdefault(base, {})
            ent["weight" if mm.group(2) == "weight" else ("offset" if mm.group(2) == "weight_offset" else "scale")] = t
            self._flush(base)
        for base, ent in list(self._pending.items()):   # int8 without offset, fp8 without scale
            if "weight" in ent:
                self._route(base, ent["weight"], ent.get("scale"), ent.get("offset"))
        self._pending.clear()
        self.model.process_weights_after_loading()
        return self.loaded

    def _flush(self, base):
        ent = self._pending[base]
        w = ent.get("weight")
        if w is None or "scale" not in ent:
            return
        if w.dtype == torch.int8 and "offset" not in ent and self._expects_offset:
            return
        self._route(base, w, ent["scale"], ent.get("offset"))
        del self._pending[base]

    _expects_offset = False


def _draw_shared(moe, pname: str, p, gen, std):
    """The whole shared-expert tensor (merged gate/up for ``w13``, down for ``w2``) as the random initialisation draws it
    for a model that keeps the shared expert on every rank; e4m3 models get (bytes, scale blocks)."""
    cfg = moe.cfg
    I, H = cfg.moe_intermediate_size * cfg.n_shared_experts, cfg.hidden_size
    prefix = pname.rsplit(".", 1)[0]
    which = "gate_up_proj" if pname.endswith("w13") else "down_proj"
    g = gen(p.device, f"{prefix}.shared_experts.{which}.weight")
    w = torch.randn((2 * I, H) if which == "gate_up_proj" else (H, I), generator=g, device=g.device, dtype=torch.float32) * std
    if p.dtype == FP8:
        assert cfg.moe_intermediate_size % 128 == 0, "e4m3 shared-expert pieces must be aligned to the scale blocks"
        return quant_weight_fp8_block_ref(w)
    return w, None


def iter_safetensors(model_dir: str):
    """Yield (name, tensor) from every *.safetensors shard of a HF checkpoint directory."""
    from safetensors import safe_open   # optional dependency, only needed for real checkpoints

    for f in sorted(Path(model_dir).glob("*.safetensors")):
        with safe_open(str(f), framework="pt") as sf:
            for k in sf.keys():
                yield k, sf.get_tensor(k)


def load_quant_description(model_dir: str) -> dict:
    """``quant_model_description.json`` of the int8 compressed-tensors layout
    (omni/quantization/compressed_tensors/compressed_tensors.py:66)."""
    p = Path(model_dir) / "quant_model_description.json"
    return json.loads(p.read_text()) if p.exists() else {}


@torch.no_grad()
def init_random_weights(model, seed: int = 0, std: float = 0.02) -> None:
    """Random N(0, std) initialisation (norm weights = 1, biases = 0).  Every tensor gets its own generator
    seeded from (seed, parameter name) and every routed expert from (seed, layer, logical expert id), so the
    weights do not depend on how many ranks the experts are sharded over: a 2-rank model is the same model as
    the 1-rank one.  Quantised tensors are drawn in fp32 and block-quantised on their device."""
    import os
    import zlib

    params = dict(model.named_parameters())
    # OMNI_INIT_ON_HOST=1 draws and quantises on the CPU and copies the result over: a handful of memcpys per
    # tensor instead of a dozen small kernels (for tiny models whose first launches should be the model's own)
    host_init = os.environ.get("OMNI_INIT_ON_HOST", "0") == "1"

    def gen(dev, *key):
        if host_init:
            dev = "cpu"
        g = torch.Generator(device=dev)
        g.manual_seed((seed * 1000003 + zlib.crc32("/".join(str(k) for k in key).encode())) % (2 ** 63 - 1))
        return g

    def fill(p, sp, g):
        if host_init:
            full = getattr(p, "tp_full_shape", None)
            w = torch.randn(tuple(full) if full is not None else tuple(p.shape), generator=g, dtype=torch.float32) * std
            s_ = None
            if p.dtype == FP8:
                w, s_ = quant_weight_fp8_block_ref(w)
            if full is not None:
                w = p.tp_slice_fn(w)
                s_ = sp.tp_slice_fn(s_) if s_ is not None else None
            p.copy_(w.to(p.dtype))
            if s_ is not None:
                sp.copy_(s_)
            return
        full = getattr(p, "tp_full_shape", None)
        if full is not None:
            # tensor-parallel shard: draw the whole tensor (so that the sharded model is the unsharded one), keep this
            # rank's slice; e4m3 tensors are quantised whole and their scale blocks sliced alongside
            w = torch.randn(full, generator=g, device=p.device, dtype=torch.float32) * std
            if p.dtype == FP8:
                q, s_ = quant_weight_fp8_block_ref(w)
                p.copy_(p.tp_slice_fn(q))
                sp.copy_(sp.tp_slice_fn(s_))
            else:
                p.copy_(p.tp_slice_fn(w))
            return
        if p.dtype == FP8:
            w = torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * std
            q, s = quant_weight_fp8_block_ref(w)
            p.copy_(q)
            sp.copy_(s)
        elif p.numel() > (1 << 28):
            flat = p.view(-1)
            step = 1 << 26
            for i in range(0, flat.numel(), step):
                n = min(step, flat.numel() - i)
                flat[i:i + n].copy_(torch.randn(n, generator=g, device=p.device, dtype=torch.float32) * std)
        else:
            p.copy_(torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * std)

    expert_params = {}
    for mname, mod in model.named_modules():
        if mod.__class__.__name__ == "MoELayer":
            for pn in ("w13", "w2"):
                expert_params[f"{mname}.{pn}" if mname else pn] = mod
    for name, p in params.items():
        if name.endswith(("_scale", "weight_scale")):
            continue
        if name in expert_params:
            mod = expert_params[name]
            sp = params.get(name + "_scale")
            shared_full = None
            for slot in range(p.shape[0]):
                logical = mod.logical_of_slot(slot) if mod.planner is None else mod.planner.logical_of_slot(mod.moe_index, slot)
                if logical is None:
                    continue                      # an unused slot of a shared-expert rank stays zero
                if isinstance(logical, tuple):
                    # piece of the shared expert: draw the tensor the model without shared-expert ranks would hold under
                    # its name there, quantise it whole, keep this piece
                    if shared_full is None:
                        shared_full = _draw_shared(mod, name, p, gen, std)
                    q, s_ = shared_full
                    I, j = mod.cfg.moe_intermediate_size, logical[1]
                    ns = mod.shared_pieces
                    if name.endswith("w13"):
                        p[slot].copy_(torch.cat([q[j * I:(j + 1) * I], q[(ns + j) * I:(ns + j + 1) * I]], 0))
                        if s_ is not None:
                            sp[slot].copy_(torch.cat([s_[j * I // 128:(j + 1) * I // 128],
                                                      s_[(ns + j) * I // 128:(ns + j + 1) * I // 128]], 0))
                    else:
                        p[slot].copy_(q[:, j * I:(j + 1) * I])
                        if s_ is not None:
                            sp[slot].copy_(s_[:, j * I // 128:(j + 1) * I // 128])
                    continue
                g = gen(p.device, name, "expert", logical)
                fill(p[slot], sp[slot] if sp is not None else None, g)
            continue
        g = gen(p.device, name)
        if "norm" in name and p.dim() == 1:
            p.fill_(1.0)
        elif name.endswith("bias") and p.dim() == 1 and "e_score" not in name:
            p.zero_()
        elif name.endswith("e_score_correction_bias"):
            p.copy_(torch.randn(p.shape, generator=g, device=g.device) * 0.01)
        else:
            fill(p, params.get(name + "_scale"), g)
    model.process_weights_after_loading()
