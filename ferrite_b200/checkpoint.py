"""Hugging Face checkpoints for the decode path: config.json and model*.safetensors read as the reference reads them
(models/llama.py:376-427 `fuse`, :545-570 `config`, :572-604 `load`; models/gpt2.py:34-47 `safetensors`, `tensor_bits`),
under the reference's weight names (qkv_proj = q | k | v side by side, gate_up_proj = gate | up, everything as x @ w
takes it, a mixture's experts as batches, Qwen3's q/k norms as a batch of every head's).

The file is mapped, never read whole.  A weight is a small recipe over the file's tensors (transpose, side by side, a
batch) that is carried out either on the host in numpy (`bits()`: what the oracle and small models use) or on the GPU
(`device(rt)`: every piece is copied up as it lies in the file and transposed / joined there by this library's strided
copy kernel, so an 8 B-parameter model's transposes cost no host time); `llama.upload` then casts each matrix to its
block-float format on the device.  Covered: Llama / SmolLM / Qwen3 dense models and Mixtral- and Qwen3-style mixtures
(BF16 or F32 tensors).  Not covered, and refused by name: Gated DeltaNet blocks, gated attention, biases, MXFP4 experts.
"""
import json
import os
import re
import struct

import numpy as np

from . import llama


def safetensors(path):
    """A safetensors file: its JSON header (each tensor's dtype, shape and byte range) and its data, mapped
    (models/gpt2.py:34-38)."""
    with open(path, "rb") as f:
        size = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(size))
    return header, np.memmap(path, np.uint8, "r", offset=8 + size)


def bf16_bits(a):
    """float32 values as bf16 bits, rounded to nearest even (models/gpt2.py:16-18)."""
    b = np.ascontiguousarray(a, np.float32).view(np.uint32)
    return ((b + (0x7FFF + (b >> 16 & 1))) >> 16).astype(np.uint16)


class Weight:
    """A weight made when it is wanted (models/llama.py:530-535): bits() its bf16 bits as x @ w takes them (numpy),
    values() the same as float32, device(rt) the same on the GPU as a bf16 Tensor."""

    def __init__(self, bits, device=None):
        self.bits, self._device = bits, device

    def values(self):
        return (self.bits().astype(np.uint32) << 16).view(np.float32)

    def device(self, rt):
        from .tensor import Tensor
        if self._device is not None:
            return self._device(rt)
        b = self.bits()
        return Tensor.frombytes(rt, *b.shape[-2:], b.tobytes(), b.shape[0] if b.ndim == 3 else 1)


def leaf(data, t, turn=False):
    """One tensor of a file (models/gpt2.py:40-47): BF16 as it is, F32 rounded; a vector as one row; turn: transposed."""
    def bits():
        raw = data[t["data_offsets"][0]:t["data_offsets"][1]]
        if t["dtype"] == "F32":
            b = bf16_bits(raw.view(np.float32))
        else:
            assert t["dtype"] == "BF16", f"{t['dtype']} tensors are not read (BF16 or F32)"
            b = raw.view(np.uint16)
        b = b.reshape(t["shape"] if len(t["shape"]) >= 2 else (1, -1))
        return np.ascontiguousarray(np.swapaxes(b, -1, -2)) if turn else np.ascontiguousarray(b)

    def device(rt):
        from .tensor import Tensor
        shape = t["shape"] if len(t["shape"]) >= 2 else [1] + list(t["shape"] or [1])
        raw = data[t["data_offsets"][0]:t["data_offsets"][1]]
        if t["dtype"] == "F32":  # rounded on the device: an fp32 upload, then a cast
            x = Tensor.frombytes(rt, shape[-2], shape[-1], raw.tobytes(), int(np.prod(shape[:-2])), "fp32").bfloat16().realize()
        else:
            assert t["dtype"] == "BF16", f"{t['dtype']} tensors are not read (BF16 or F32)"
            x = Tensor.frombytes(rt, shape[-2], shape[-1], raw.tobytes(), int(np.prod(shape[:-2])))
        return (x.T + 0).realize() if turn else x
    return Weight(bits, device)


def join(*ws):
    """Matrices side by side (q | k | v; gate | up)."""
    return Weight(lambda: np.ascontiguousarray(np.concatenate([w.bits() for w in ws], -1)),
                  lambda rt: (lambda xs: xs[0].cat(*xs[1:], axis=2))([w.device(rt) for w in ws]))


def stack(ws):
    """Matrices as a batch (a mixture's experts; every head's norm)."""
    return Weight(lambda: np.stack([w.bits() for w in ws]),
                  lambda rt: (lambda xs: xs[0].cat(*xs[1:], axis=0))([w.device(rt) for w in ws]))


def read_json(path):
    with open(path, encoding="utf-8") as f:
        return json.load(f)


def config(folder, places=4096):
    """A model's config.json as a decode-path config (models/llama.py:545-570), for the families covered here."""
    j = read_json(os.path.join(folder, "config.json"))
    j = j.get("text_config", j)
    rope = j.get("rope_parameters") or (j.get("rope_scaling") or {}) | {"rope_theta": j["rope_theta"]}
    theta, kind = rope.pop("rope_theta"), rope.pop("type", None)
    rope.setdefault("rope_type", kind or "default")
    assert rope["rope_type"] in ("default", "llama3"), f"RoPE scaling {rope}: not covered by this decode path"
    assert not j.get("linear_num_key_heads") and not j.get("attn_output_gate"), "Gated DeltaNet / gated attention models are not covered"
    experts = j.get("num_experts") or j.get("num_local_experts") or 0
    return llama.model(dim=j["hidden_size"], heads=j["num_attention_heads"], kv=j["num_key_value_heads"], layers=j["num_hidden_layers"],
                       eps=j["rms_norm_eps"], theta=theta, places=min(j["max_position_embeddings"], places), vocab=j["vocab_size"],
                       ffn=j.get("intermediate_size"), head_dim=j.get("head_dim"), rope=rope if rope["rope_type"] != "default" else None,
                       sliding=j.get("sliding_window") if j.get("use_sliding_window", True) else None, experts=experts,
                       k=j.get("num_experts_per_tok") or 0, moe=j.get("moe_intermediate_size") or (experts and j.get("intermediate_size")) or 0,
                       norm_topk=j.get("norm_topk_prob", True), tied=j.get("tie_word_embeddings", False))


def fuse(w, c):
    """Each block's q, k and v projections as one matrix, and its gate and up; a mixture's router as x @ w takes it, and
    its experts' gate | up, and downs, each a batch; Qwen3's norms of q's and k's heads as a batch of every head's
    (models/llama.py:376-427, the families covered here)."""
    for pre in sorted({k[:k.index(".", 7) + 1] for k in w if k.startswith("layers.")}):
        assert pre + "conv1d" not in w and pre + "q_proj.bias" not in w and pre + "sinks" not in w, f"{pre}: a block of a family this decode path does not cover"
        w[pre + "qkv_proj"] = join(w.pop(pre + "q_proj"), w.pop(pre + "k_proj"), w.pop(pre + "v_proj"))
        if pre + "q_norm" in w:
            q, k = w.pop(pre + "q_norm"), w.pop(pre + "k_norm")
            w[pre + "qk_norm"] = stack([q] * c.heads + [k] * c.kv)  # (this library's kernel leaves v's heads alone: no rows of 1 for them)
        router = w.pop(pre + "router") if pre + "router" in w else w.pop(pre + "gate", None)
        if router is None:  # a SwiGLU
            w[pre + "gate_up_proj"] = join(w.pop(pre + "gate_proj"), w.pop(pre + "up_proj"))
            continue
        assert pre + "experts.gate_up_proj_bias" not in w and pre + "shared_expert_gate" not in w, f"{pre}: expert biases / a shared expert are not covered"
        w[pre + "router"] = router
        n = sum(k.startswith(pre + "experts.") and k.endswith(".down_proj") for k in w)
        expert = lambda name: [w.pop(f"{pre}experts.{e}.{name}") for e in range(n)]
        gates, ups = expert("gate_proj"), expert("up_proj")
        w[pre + "experts.gate_up"], w[pre + "experts.down"] = stack([join(g, u) for g, u in zip(gates, ups)]), stack(expert("down_proj"))
    return w


def load(folder, places=4096):
    """The config, and {name: Weight} from model.safetensors or the files model.safetensors.index.json names, named
    without "model.", linear weights transposed (so x @ w), vectors as one-row matrices; the output layer is the
    embedding unless the model has its own (lm_head) (models/llama.py:572-604).  RoPE's tables (one head wide, as this
    library's kernel takes them) have a row for each of the first `places` places."""
    c = config(folder, places)
    index = os.path.join(folder, "model.safetensors.index.json")
    files = sorted(set(read_json(index)["weight_map"].values())) if os.path.exists(index) else ["model.safetensors"]
    out, tensors = {}, {}
    for file in files:
        header, data = safetensors(os.path.join(folder, file))
        tensors |= {name: (data, t) for name, t in header.items() if name != "__metadata__"}
    for full, (data, t) in tensors.items():
        name = full.removeprefix("model.").removeprefix("language_model.").removesuffix(".weight")
        for part in ("self_attn.", "mlp.", "block_sparse_moe."):
            name = name.replace(part, "")
        name = re.sub(r"(experts\.\d+)\.w([123])$", lambda m: m[1] + (".gate_proj", ".down_proj", ".up_proj")[int(m[2]) - 1], name)  # Mixtral's
        if name.startswith(("visual.", "mtp.")) or name.endswith(("_blocks", "_scales")):
            continue
        if name.startswith("layers.") and int(name.split(".")[1]) >= c.layers:
            continue  # (a config cut to its first blocks)
        # a linear layer's matrix is stored (out x in): transposed for x @ w; a mixture's router ("gate") likewise
        turn = bool(re.search(r"_proj$|^lm_head$|\.gate$|\.router$", name)) and len(t["shape"]) == 2
        out[name] = leaf(data, t, turn)
    out["embed"] = out.pop("embed_tokens")
    own = out.pop("lm_head", None)
    embed = out["embed"]
    out["embed.T"] = own or Weight(lambda: np.ascontiguousarray(embed.bits().T), lambda rt: (embed.device(rt).T + 0).realize())
    cos, sin = llama.rotary(c, c.places)
    out["cos"], out["sin"] = Weight(lambda: bf16_bits(cos)), Weight(lambda: bf16_bits(sin))
    return c, fuse(out, c)


def save(folder, c, weights, dtype="BF16", shards=1):
    """Write {name: float32 array of bf16 values} (this library's fused names, as oracle.llama.synthetic draws them) as
    a Hugging Face checkpoint: config.json and model.safetensors (or `shards` files and their index), the linear weights
    un-fused and stored (out x in) under the hub's names.  For tests of `load` and for handing a model made here to other
    tools; the reference has no counterpart (it only reads checkpoints)."""
    os.makedirs(folder, exist_ok=True)
    hd, H, KV = llama.head(c), c.heads, c.kv
    t = {"model.embed_tokens.weight": weights["embed"], "model.norm.weight": weights["norm"].reshape(-1)}
    if not c.tied:
        t["lm_head.weight"] = np.ascontiguousarray(weights["embed.T"].T)
    for l in range(c.layers):
        p, q = f"layers.{l}.", f"model.layers.{l}."
        qkv = weights[p + "qkv_proj"]
        for name, cols in (("q_proj", slice(0, H * hd)), ("k_proj", slice(H * hd, (H + KV) * hd)), ("v_proj", slice((H + KV) * hd, None))):
            t[f"{q}self_attn.{name}.weight"] = np.ascontiguousarray(qkv[:, cols].T)
        t[q + "self_attn.o_proj.weight"] = np.ascontiguousarray(weights[p + "o_proj"].T)
        t[q + "input_layernorm.weight"], t[q + "post_attention_layernorm.weight"] = weights[p + "input_layernorm"].reshape(-1), weights[p + "post_attention_layernorm"].reshape(-1)
        if p + "qk_norm" in weights:
            t[q + "self_attn.q_norm.weight"], t[q + "self_attn.k_norm.weight"] = weights[p + "qk_norm"][0].reshape(-1), weights[p + "qk_norm"][H].reshape(-1)
        if p + "router" in weights:
            t[q + "mlp.gate.weight"] = np.ascontiguousarray(weights[p + "router"].T)
            m = weights[p + "experts.down"].shape[1]
            for e in range(c.experts):
                gu = weights[p + "experts.gate_up"][e]
                t[f"{q}mlp.experts.{e}.gate_proj.weight"], t[f"{q}mlp.experts.{e}.up_proj.weight"] = np.ascontiguousarray(gu[:, :m].T), np.ascontiguousarray(gu[:, m:].T)
                t[f"{q}mlp.experts.{e}.down_proj.weight"] = np.ascontiguousarray(weights[p + "experts.down"][e].T)
        else:
            gu, m = weights[p + "gate_up_proj"], weights[p + "down_proj"].shape[0]
            t[q + "mlp.gate_proj.weight"], t[q + "mlp.up_proj.weight"] = np.ascontiguousarray(gu[:, :m].T), np.ascontiguousarray(gu[:, m:].T)
            t[q + "mlp.down_proj.weight"] = np.ascontiguousarray(weights[p + "down_proj"].T)
    cfg = {"hidden_size": c.dim, "num_attention_heads": H, "num_key_value_heads": KV, "num_hidden_layers": c.layers, "rms_norm_eps": c.eps,
           "rope_theta": c.theta, "max_position_embeddings": c.places, "vocab_size": c.vocab, "intermediate_size": c.ffn or c.moe,
           "head_dim": c.head_dim, "tie_word_embeddings": bool(c.tied)}
    if c.rope:
        cfg["rope_scaling"] = c.rope
    if c.experts:
        cfg |= {"num_experts": c.experts, "num_experts_per_tok": c.k, "moe_intermediate_size": c.moe, "norm_topk_prob": c.norm_topk}
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    names = sorted(t)
    per = -(-len(names) // shards)
    index = {}
    for s in range(shards):
        part = names[s * per:(s + 1) * per]
        file = "model.safetensors" if shards == 1 else f"model-{s + 1:05d}-of-{shards:05d}.safetensors"
        header, blobs, at = {}, [], 0
        for name in part:
            a = np.asarray(t[name], np.float32)
            raw = (bf16_bits(a) if dtype == "BF16" else a).tobytes()
            header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
            blobs.append(raw)
            at += len(raw)
            index[name] = file
        head = json.dumps(header).encode()
        head += b" " * (-len(head) % 8)
        with open(os.path.join(folder, file), "wb") as f:
            f.write(struct.pack("<Q", len(head)) + head + b"".join(blobs))
    if shards > 1:
        with open(os.path.join(folder, "model.safetensors.index.json"), "w") as f:
            json.dump({"weight_map": index}, f)
