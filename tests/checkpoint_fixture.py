"""Test helper: a LeRobot-layout PI0.5 checkpoint (the tensor names, [out, in] orientation and
unfolded `w` RMSNorm parameters a real file has) written from the oracle's synthetic weights,
so that loading it must reproduce those weights."""
import numpy as np

from oracle import pi05_oracle as O

ROOT = "paligemma_with_expert"


def _bits(x):
    return O.bf16_bits(np.asarray(x, dtype=np.float32))


def lerobot_tensors(cfg, seed, *, norm_seed=None, wrap_prefix=False, embedding_alias=False):
    """name -> uint16 bf16 array in checkpoint layout. `norm_seed` None: RMSNorm `w` = 0 and
    LayerNorm gamma 1 / beta 0 (the loaded model then equals the synthetic one); else small
    seeded values for every norm parameter."""
    w = O.SyntheticWeights(cfg, seed)
    rng = np.random.default_rng(norm_seed) if norm_seed is not None else None
    out = {}

    def linear(dst, src, bias):
        out[dst + ".weight"] = _bits(w.get(src + ".weight").T)
        if bias:
            out[dst + ".bias"] = _bits(w.get(src + ".bias"))

    def norm_values(width, centre):
        if rng is None:
            return np.full(width, centre, np.float32)
        return (centre + rng.uniform(-0.25, 0.25, width)).astype(np.float32)

    def layer_norm(dst, width):
        out[dst + ".weight"] = _bits(norm_values(width, 1.0))
        out[dst + ".bias"] = _bits(norm_values(width, 0.0))

    vw = cfg.vision_width
    vp = f"{ROOT}.paligemma.model.vision_tower.vision_model"
    for i in range(cfg.vision_depth):
        p, s = f"{vp}.encoder.layers.{i}", f"vision.{i}"
        layer_norm(p + ".layer_norm1", vw)
        layer_norm(p + ".layer_norm2", vw)
        for dst, src in (("self_attn.q_proj", "q"), ("self_attn.k_proj", "k"), ("self_attn.v_proj", "v"),
                         ("self_attn.out_proj", "o"), ("mlp.fc1", "fc1"), ("mlp.fc2", "fc2")):
            linear(f"{p}.{dst}", f"{s}.{src}", True)
    patch = w.get("vision.patch_embedding.weight").T  # [vw, 3 * p * p]
    out[f"{vp}.embeddings.patch_embedding.weight"] = _bits(patch).reshape(vw, 3, cfg.patch_size, cfg.patch_size)
    out[f"{vp}.embeddings.patch_embedding.bias"] = _bits(w.get("vision.patch_embedding.bias"))
    out[f"{vp}.embeddings.position_embedding.weight"] = _bits(w.get("vision.position_embedding"))
    layer_norm(f"{vp}.post_layernorm", vw)
    linear(f"{ROOT}.paligemma.model.multi_modal_projector.linear", "vision.projector", True)
    name = f"{ROOT}.paligemma.lm_head.weight" if embedding_alias else \
        f"{ROOT}.paligemma.model.language_model.embed_tokens.weight"
    out[name] = _bits(w.get("token_embedding"))

    def gemma(p, s):
        for dst, src in (("self_attn.q_proj", "q"), ("self_attn.k_proj", "k"), ("self_attn.v_proj", "v"),
                         ("self_attn.o_proj", "o"), ("mlp.gate_proj", "gate"), ("mlp.up_proj", "up"),
                         ("mlp.down_proj", "down")):
            linear(f"{p}.{dst}", f"{s}.{src}", False)

    lp = f"{ROOT}.paligemma.model.language_model"
    for i in range(cfg.language.depth):
        p = f"{lp}.layers.{i}"
        gemma(p, f"language.{i}")
        out[p + ".input_layernorm.weight"] = _bits(norm_values(cfg.language.width, 0.0))
        out[p + ".post_attention_layernorm.weight"] = _bits(norm_values(cfg.language.width, 0.0))
    out[f"{lp}.norm.weight"] = _bits(norm_values(cfg.language.width, 0.0))
    ap = f"{ROOT}.gemma_expert.model"
    for i in range(cfg.action_expert.depth):
        p = f"{ap}.layers.{i}"
        gemma(p, f"action.{i}")
        linear(p + ".input_layernorm.dense", f"action.{i}.input_style", True)
        linear(p + ".post_attention_layernorm.dense", f"action.{i}.post_style", True)
    linear(f"{ap}.norm.dense", "action.final_style", True)
    linear("action_in_proj", "action_in", True)
    linear("action_out_proj", "action_out", True)
    linear("time_mlp_in", "time_mlp_in", True)
    linear("time_mlp_out", "time_mlp_out", True)
    if wrap_prefix:
        out = {"model." + k: v for k, v in out.items()}
    return out


def expected_table(cfg, seed, tensors):
    """What the loader must produce for `lerobot_tensors(cfg, seed, ...)`: the synthetic tensors,
    with q/k/v and gate/up of the language model scaled per input channel by bf16(1 + w) in
    float32, and the LayerNorm parameters passed through. Values as float32 arrays."""
    tensors = {(k[len("model."):] if k.startswith("model." + ROOT) else k): v for k, v in tensors.items()}
    w = O.SyntheticWeights(cfg, seed)
    table = {name: w.get(name) for name in w.layout if name != "__total__"}
    lp = f"{ROOT}.paligemma.model.language_model"
    for i in range(cfg.language.depth):
        for norm, parts in (("input_layernorm", ("q", "k", "v")), ("post_attention_layernorm", ("gate", "up"))):
            raw = O.bf16_from_bits(tensors[f"{lp}.layers.{i}.{norm}.weight"])
            scale = O.round_bf16(raw + np.float32(1.0))
            for part in parts:
                table[f"language.{i}.{part}.weight"] = table[f"language.{i}.{part}.weight"] * scale[:, None]
    vp = f"{ROOT}.paligemma.model.vision_tower.vision_model"
    for i in range(cfg.vision_depth):
        for n, src in (("norm1", "layer_norm1"), ("norm2", "layer_norm2")):
            for part in ("weight", "bias"):
                table[f"vision.{i}.{n}.{part}"] = O.bf16_from_bits(tensors[f"{vp}.encoder.layers.{i}.{src}.{part}"])
    for part in ("weight", "bias"):
        table[f"vision.post_norm.{part}"] = O.bf16_from_bits(tensors[f"{vp}.post_layernorm.{part}"])
    return table


def write_checkpoint(path, tensors, shards=1):
    """`path` directory: model.safetensors, or `shards` files plus the index json."""
    import json
    import os
    from apxinf_b200 import checkpoint as ck
    os.makedirs(path, exist_ok=True)
    arrays = {k: ck.HostArray("bf16", v) for k, v in tensors.items()}
    if shards == 1:
        ck.save_file(os.path.join(path, "model.safetensors"), arrays)
        return
    names = list(arrays)
    weight_map = {}
    for s in range(shards):
        part = names[s::shards]
        file = f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        ck.save_file(os.path.join(path, file), {k: arrays[k] for k in part})
        weight_map.update({k: file for k in part})
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as handle:
        json.dump({"metadata": {}, "weight_map": weight_map}, handle)
