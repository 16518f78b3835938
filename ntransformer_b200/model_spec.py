"""Llama-3 shapes and per-tensor quantisation mixes of the benchmark configs.

The Q4_K_M recipe follows llama.cpp ftype 15 as SURVEY §8d states it: everything Q4_K except attn_v and
ffn_down, which are Q6_K on layers with  i < L/8  or  i >= 7L/8  or  (i - L/8) % 3 == 2 ;  on the 70B shape the
remaining attn_v are Q5_K ; output.weight is Q6_K, token_embd Q4_K, norms F32."""
from __future__ import annotations

from dataclasses import dataclass, asdict

from .dtypes import DType, dtype_row_size


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    max_seq_len: int = 4096
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    bos_token_id: int = 128000
    eos_token_id: int = 128009

    def dict(self):
        return asdict(self)


LLAMA3_8B = LlamaConfig()
LLAMA3_70B = LlamaConfig(hidden_size=8192, intermediate_size=28672, n_layers=80, n_heads=64)
TINY = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, n_layers=3, n_heads=8, n_kv_heads=2, head_dim=64,
                   max_seq_len=128, bos_token_id=1, eos_token_id=2)

LAYER_TENSORS = ("attn_norm", "attn_q", "attn_k", "attn_v", "attn_output", "ffn_norm", "ffn_gate", "ffn_up", "ffn_down")


def use_more_bits(i: int, n: int) -> bool:
    return i < n // 8 or i >= 7 * n // 8 or (i - n // 8) % 3 == 2


def tensor_dtype(mix: str, name: str, layer: int, n_layers: int, big: bool) -> DType:
    """dtype of GGUF tensor `name` ('attn_q', 'output', 'token_embd', ...) under quantisation mix `mix`."""
    if name.endswith("norm"):
        return DType.F32
    mix = mix.upper()
    if mix == "Q4_K_M":
        if name == "output":
            return DType.Q6_K
        if name == "token_embd":
            return DType.Q4_K_M
        if name in ("attn_v", "ffn_down"):
            if use_more_bits(layer, n_layers):
                return DType.Q6_K
            return DType.Q5_K if (big and name == "attn_v") else DType.Q4_K_M
        return DType.Q4_K_M
    return {"Q8_0": DType.Q8_0, "Q4_0": DType.Q4_0, "Q6_K": DType.Q6_K, "Q5_K": DType.Q5_K, "Q4_K": DType.Q4_K_M,
            "F16": DType.F16, "F32": DType.F32}[mix]


def tensor_table(cfg: LlamaConfig, mix: str, tp_rank: int = 0, tp_size: int = 1):
    """[(gguf_name, dtype, rows, cols)] for this rank's shard, in file order."""
    big = cfg.n_layers >= 64
    hd, h = cfg.head_dim, cfg.hidden_size
    nh, nkv, inter = cfg.n_heads // tp_size, cfg.n_kv_heads // tp_size, cfg.intermediate_size // tp_size
    vl = -(-cfg.vocab_size // tp_size)
    vrows = cfg.vocab_size if tp_size == 1 else max(0, min(vl, cfg.vocab_size - tp_rank * vl))
    t = [("token_embd.weight", tensor_dtype(mix, "token_embd", 0, cfg.n_layers, big), cfg.vocab_size, h),
         ("output_norm.weight", DType.F32, 1, h),
         ("output.weight", tensor_dtype(mix, "output", 0, cfg.n_layers, big), vrows, h)]
    shapes = {"attn_norm": (1, h), "ffn_norm": (1, h), "attn_q": (nh * hd, h), "attn_k": (nkv * hd, h), "attn_v": (nkv * hd, h),
              "attn_output": (h, nh * hd), "ffn_gate": (inter, h), "ffn_up": (inter, h), "ffn_down": (h, inter)}
    for i in range(cfg.n_layers):
        for n in LAYER_TENSORS:
            r, c = shapes[n]
            t.append((f"blk.{i}.{n}.weight", tensor_dtype(mix, n, i, cfg.n_layers, big), r, c))
    return t


def bytes_per_token(cfg: LlamaConfig, mix: str, ctx: int, tp_size: int = 1) -> int:
    """Algorithmic bytes read per decoded token: 7 projections x L + output.weight + norms + KV."""
    b = 0
    for name, dt, r, c in tensor_table(cfg, mix, 0, tp_size):
        if name == "token_embd.weight":
            continue
        b += r * (c * 4 if dt == DType.F32 and r == 1 else dtype_row_size(dt, c))
    return b + 2 * cfg.n_layers * ctx * (cfg.n_kv_heads // tp_size) * cfg.head_dim * 2


# ---- Zelunex (layer-spec family, model folders): synthetic configurations and random device weights for benchmarks ----
def zelunex_config(vocab=32000, width=4096, n_layers=4, heads=32, kv_heads=8, dim=128, vdim=128, ff=14336, window=1024, keep_first=4,
                   softcap=30.0, eps=1e-5, residual_mult=0.5, share=None):
    """The family's config.json as a dict.  share: {layer: earlier layer whose tensors it reads}."""
    share = share or {}
    layers = []
    for i in range(n_layers):
        e = {"type": "attention",
             "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "softcap": softcap,
                       "mask": {"size": window, "keep_first": keep_first}},
             "mlp": {"kind": "dense", "ff": ff} if ff else None}
        if i in share:
            e["weights_of"] = share[i]
        layers.append(e)
    return {"architecture": "Zelunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": residual_mult, "layers": layers}


def zelunex_random_tensors(config: dict, seed: int = 1234, device="cuda", dtype=None):
    """Checkpoint name -> random CUDA tensor (matrices `dtype`, default bfloat16; gain vectors float32)."""
    import torch

    dtype = dtype or torch.bfloat16
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W = config["width"]

    def mat(rows, cols):
        return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * cols ** -0.5).to(dtype)

    def vec(n):
        return 1.0 + 0.1 * torch.randn(n, generator=g, device=device, dtype=torch.float32)

    t = {"embed": mat(config["vocab"], W) * W ** 0.5, "final.norm": vec(W), "head": mat(config["vocab"], W)}
    for i, e in enumerate(config["layers"]):
        if "weights_of" in e:
            continue
        m, p = e["mixer"], "l%d." % i
        t[p + "norm1"] = vec(W)
        t[p + "mix.q"] = mat(m["heads"] * m["dim"], W)
        t[p + "mix.k"] = mat(m["kv_heads"] * m["dim"], W)
        t[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], W)
        t[p + "mix.q.norm"] = vec(m["heads"] * m["dim"])
        t[p + "mix.k.norm"] = vec(m["kv_heads"] * m["dim"])
        t[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        t[p + "ls1"] = vec(W)
        if e.get("mlp"):
            t[p + "mlp.gate"] = mat(e["mlp"]["ff"], W)
            t[p + "mlp.up"] = mat(e["mlp"]["ff"], W)
            t[p + "mlp.down"] = mat(W, e["mlp"]["ff"])
            t[p + "ls2"] = vec(W)
    return t


# ---- Vebotar (layer-spec family, model folders): synthetic configurations and random device weights for benchmarks ----
def vebotar_config(vocab=32000, width=4096, n_layers=4, heads=32, kv_heads=8, dim=64, vdim=128, chunk=1024, rot_dims=32, rot_base=500000.0,
                   scaling=(4.0, 8192, 32.0, 1.0), diff=0.3, experts=8, top=2, ff=4096, shared_ff=4096, streams=2, embed_scale=1.0, eps=1e-5,
                   kv_from=None):
    """The family's config.json as a dict.  dim is the width of ONE score map (a head has two).  kv_from: {layer: earlier layer whose
    cache it reads}.  scaling: (factor, original, fast, slow) of the long-context frequency blend, or None."""
    kv_from = kv_from or {}
    layers = []
    for i in range(n_layers):
        m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "diff": diff, "mask": {"size": chunk},
             "rot": {"dims": rot_dims, "base": rot_base}}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
        if i in kv_from:
            m["kv_from"] = kv_from[i]
        mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
        if shared_ff:
            mlp["shared"] = {"ff": shared_ff}
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Vebotar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    return cfg


def vebotar_random_tensors(config: dict, seed: int = 1234, device="cuda", dtype=None):
    """Checkpoint name -> random CUDA tensor (matrices `dtype`, default bfloat16; gains, lambda vectors, stream tables, router float32)."""
    import torch

    dtype = dtype or torch.bfloat16
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W, S = config["width"], config.get("streams", 0)

    def mat(rows, cols, dt=dtype):
        return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * cols ** -0.5).to(dt)

    def vec(n, mean=1.0, std=0.1):
        return mean + std * torch.randn(n, generator=g, device=device, dtype=torch.float32)

    t = {"embed": mat(config["vocab"], W) * W ** 0.5, "final.norm": vec(W), "head": mat(config["vocab"], W)}
    for i, e in enumerate(config["layers"]):
        m, p = e["mixer"], "l%d." % i
        t[p + "norm1"] = vec(W)
        t[p + "mix.q"] = mat(m["heads"] * 2 * m["dim"], W)
        if "kv_from" not in m:
            t[p + "mix.k"] = mat(m["kv_heads"] * 2 * m["dim"], W)
            t[p + "mix.v"] = mat(m["kv_heads"] * m["vdim"], W)
        for n in ("lq1", "lk1", "lq2", "lk2"):
            t[p + "mix." + n] = vec(m["dim"], 0.0, 0.1)
        t[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        subs = ["hc1."] + (["hc2."] if e.get("mlp") else [])
        for q in subs if S else []:
            t[p + q + "in"] = vec(S, 1.0 / S, 0.05)
            t[p + q + "out"] = vec(S, 1.0, 0.05)
            t[p + q + "mix"] = torch.eye(S, device=device) + 0.05 * torch.randn(S, S, generator=g, device=device)
        if e.get("mlp"):
            mlp = e["mlp"]
            t[p + "norm2"] = vec(W)
            t[p + "mlp.router"] = mat(mlp["router"]["experts"], W, torch.float32)
            for x in range(mlp["router"]["experts"]):
                t[p + "mlp.e%d.up" % x] = mat(mlp["expert"]["ff"], W)
                t[p + "mlp.e%d.down" % x] = mat(W, mlp["expert"]["ff"])
            if mlp.get("shared"):
                t[p + "mlp.shared.up"] = mat(mlp["shared"]["ff"], W)
                t[p + "mlp.shared.down"] = mat(W, mlp["shared"]["ff"])
                t[p + "mlp.shared.sg"] = mat(1, W, torch.float32)
    return t


# ---- Tanolorn (layer-spec family, model folders): synthetic configurations and random device weights for benchmarks ----
def tanolorn_config(vocab=32000, width=4096, pattern=("mamba2", "latent_attention", "mamba2", "latent_attention"), kv_from=None, mlp=("dense", "moe", "moe", "moe"),
                    heads=32, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512, rot_base=10000.0,
                    s_heads=64, s_vdim=64, state=128, groups=8, conv=4, norm_groups=8, ff=8192, experts=16, top=4, eff=1408, route_groups=(4, 2), side=256,
                    eps=1e-6):
    """The family's config.json as a dict.  pattern: mixer type per layer; mlp: feed-forward kind per layer ("dense", "moe" or None);
    kv_from: {layer: earlier latent-attention layer whose cache rows it reads}; route_groups: (count, keep) or None; side: width of the
    per-layer token input (0: none)."""
    kv_from = kv_from or {}
    layers = []
    for i, typ in enumerate(pattern):
        if typ == "latent_attention":
            m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": (dim + rot_dim) ** -0.5,
                 "rot": {"dims": rot_dim, "base": rot_base}}
            if i in kv_from:
                m["kv_from"] = kv_from[i]
        else:
            m = {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}
        k = mlp[i % len(mlp)]
        if k == "dense":
            f = {"kind": "dense", "ff": ff}
        elif k == "moe":
            r = {"experts": experts, "top": top}
            if route_groups:
                r["groups"] = {"count": route_groups[0], "keep": route_groups[1]}
            f = {"kind": "moe", "expert": {"ff": eff}, "router": r}
        else:
            f = None
        layers.append({"type": typ, "mixer": m, "mlp": f})
    cfg = {"architecture": "Tanolorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def tanolorn_random_tensors(config: dict, seed: int = 1234, device="cuda", dtype=None):
    """Checkpoint name -> random CUDA tensor (matrices `dtype`, default bfloat16; gains, biases, convolution taps, scan constants, router
    rows and the choice correction float32)."""
    import math

    import torch

    dtype = dtype or torch.bfloat16
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W, side = config["width"], (config.get("token_side") or {}).get("dim", 0)
    n_layers = len(config["layers"])

    def mat(rows, cols, dt=dtype):
        return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * cols ** -0.5).to(dt)

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g, device=device, dtype=torch.float32)

    def uni(n, lo, hi):
        return lo + (hi - lo) * torch.rand(n, generator=g, device=device, dtype=torch.float32)

    t = {"embed": mat(config["vocab"], W) * W ** 0.5, "final.norm": vec(W), "head": mat(config["vocab"], W)}
    if side:
        t["side.embed"] = mat(config["vocab"], n_layers * side) * (n_layers * side) ** 0.5
    for i, e in enumerate(config["layers"]):
        m, p = e["mixer"], "l%d." % i
        t[p + "norm1"] = vec(W)
        if e["type"] == "latent_attention":
            t[p + "mix.dq"] = mat(m["q_rank"], W)
            t[p + "mix.dq.norm"] = vec(m["q_rank"], 1.0)
            t[p + "mix.uq"] = mat(m["heads"] * (m["dim"] + m["rot_dim"]), m["q_rank"])
            if "kv_from" not in m:
                t[p + "mix.dkv"] = mat(m["kv_rank"] + m["rot_dim"], W)
                t[p + "mix.dkv.norm"] = vec(m["kv_rank"], 1.0)
            t[p + "mix.uk"] = mat(m["heads"] * m["dim"], m["kv_rank"])
            t[p + "mix.uv"] = mat(m["heads"] * m["vdim"], m["kv_rank"])
            t[p + "mix.o"] = mat(W, m["heads"] * m["vdim"])
        else:
            inner = m["heads"] * m["vdim"]
            ch = inner + 2 * m["groups"] * m["state"]
            t[p + "mix.in"] = mat(inner + ch + m["heads"], W)
            t[p + "mix.conv"] = mat(ch, m["conv"], torch.float32)
            t[p + "mix.conv.b"] = vec(ch)
            t[p + "mix.dt_bias"] = uni(m["heads"], -4.0, -1.0)
            t[p + "mix.A_log"] = torch.log(uni(m["heads"], 1.0, 8.0))
            t[p + "mix.D"] = vec(m["heads"], 1.0)
            t[p + "mix.norm"] = vec(inner, 1.0)
            t[p + "mix.o"] = mat(W, inner)
        f = e.get("mlp")
        if f:
            t[p + "norm2"] = vec(W)
            if f["kind"] == "dense":
                for n, (r, c) in (("gate", (f["ff"], W)), ("up", (f["ff"], W)), ("down", (W, f["ff"]))):
                    t[p + "mlp." + n] = mat(r, c)
                    t[p + "mlp." + n + ".b"] = vec(r)
            else:
                E, eff = f["router"]["experts"], f["expert"]["ff"]
                t[p + "mlp.router"] = mat(E, W, torch.float32)
                t[p + "mlp.correction"] = vec(E, 0.0, 0.05)
                for x in range(E):
                    t[p + "mlp.e%d.gate" % x] = mat(eff, W)
                    t[p + "mlp.e%d.up" % x] = mat(eff, W)
                    t[p + "mlp.e%d.down" % x] = mat(W, eff)
        if side:
            t[p + "side.gate"] = mat(side, W)
            t[p + "side.proj"] = mat(W, side)
            t[p + "side.norm"] = vec(W, 1.0)
    return t


# ---- Savidra (layer-spec family, model folders): synthetic configurations and random device weights for benchmarks ----
def savidra_config(vocab=32000, width=2048, pattern=("parallel", "attention", "parallel", "attention"), ff=4096, v_mix=(1, 3), alpha=1.5, eps=1e-5,
                   left=None, right=None, attn=None, left_scale=1.0, right_scale=1.0):
    """The family's config.json as a dict.  pattern: mixer type per layer ("parallel": head-mixed attention beside the gated delta rule;
    "attention": sink attention); left / right / attn override the mixers' sizes; v_mix: the attention layers whose values blend with the
    first of them; ff: feed-forward width (0: none)."""
    lf = dict(heads=16, kv_heads=2, dim=128, vdim=64, conv=3, rot_dims=128, base=5e5, factor=4.0)
    lf.update(left or {})
    rt = dict(heads=16, kv_heads=16, dim=64, vdim=128, conv=4, decay_rank=64, gate_rank=64)
    rt.update(right or {})
    at = dict(heads=16, kv_heads=4, dim=128, vdim=128, rot_dims=64, base=5e5)
    at.update(attn or {})
    layers = []
    for i, typ in enumerate(pattern):
        if typ == "parallel":
            L = {"heads": lf["heads"], "kv_heads": lf["kv_heads"], "dim": lf["dim"], "vdim": lf["vdim"], "scale": lf["dim"] ** -0.5, "conv": lf["conv"],
                 "rot": {"base": lf["base"], "dims": lf["rot_dims"], "scaling": {"factor": lf["factor"]}}}
            m = {"left": L, "right": dict(rt), "left_scale": left_scale, "right_scale": right_scale}
        else:
            m = {"heads": at["heads"], "kv_heads": at["kv_heads"], "dim": at["dim"], "vdim": at["vdim"], "scale": at["dim"] ** -0.5,
                 "rot": {"base": at["base"], "dims": at["rot_dims"]}}
            if i in v_mix:
                m["v_mix"] = True
        layers.append({"type": typ, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None})
    return {"architecture": "Savidra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "postln_alpha": alpha, "layers": layers}


def savidra_random_tensors(config: dict, seed: int = 1234, device="cuda", dtype=None):
    """Checkpoint name -> random CUDA tensor (matrices `dtype`, default bfloat16; gains, biases, convolution taps, head tables and the
    delta rule's constants float32)."""
    import torch

    dtype = dtype or torch.bfloat16
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    W = config["width"]

    def mat(rows, cols, dt=dtype):
        return (torch.randn(rows, cols, generator=g, device=device, dtype=torch.float32) * cols ** -0.5).to(dt)

    def vec(n, mean=0.0, std=0.1):
        return mean + std * torch.randn(n, generator=g, device=device, dtype=torch.float32)

    def uni(n, lo, hi):
        return lo + (hi - lo) * torch.rand(n, generator=g, device=device, dtype=torch.float32)

    def taps(rows, n):
        return 0.2 + 0.5 * torch.randn(rows, n, generator=g, device=device, dtype=torch.float32)

    t = {"embed": mat(config["vocab"], W) * W ** 0.5, "final.norm": vec(W), "head": mat(config["vocab"], W)}
    for i, e in enumerate(config["layers"]):
        p = "l%d." % i
        t[p + "norm1"] = vec(W)
        t[p + "shift"] = uni(W, 0.0, 0.8)
        if e["type"] == "parallel":
            m, q = e["mixer"]["left"], p + "mix.left."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * V)):
                t[q + n] = mat(rows, W)
                t[q + n + ".b"] = vec(rows)
                t[q + n + ".conv"] = taps(rows, m["conv"])
            t[q + "q.norm"] = vec(D, 1.0)
            t[q + "k.norm"] = vec(D, 1.0)
            t[q + "talk"] = torch.eye(H, device=device) * 0.7 + 0.2 * torch.randn(H, H, generator=g, device=device)
            t[q + "temp"] = uni(H, 0.6, 1.8)
            t[q + "o"] = mat(W, H * V)
            t[q + "o.b"] = vec(W)
            m, q = e["mixer"]["right"], p + "mix.right."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                t[q + n] = mat(rows, W)
                t[q + n + ".conv"] = taps(rows, m["conv"])
            t[q + "b"] = mat(H, W)
            t[q + "A_log"] = uni(H, -3.0, 0.3)
            t[q + "norm"] = vec(V, 1.0)
            t[q + "a1"] = mat(m["decay_rank"], W)
            t[q + "a2"] = mat(H * D, m["decay_rank"])
            t[q + "dt_bias"] = uni(H * D, -4.0, -1.0)
            t[q + "g1"] = mat(m["gate_rank"], W)
            t[q + "g2"] = mat(H * V, m["gate_rank"])
            t[q + "o"] = mat(W, H * V)
        else:
            m, q = e["mixer"], p + "mix."
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[q + "q"] = mat(H * D, W)
            t[q + "k"] = mat(G * D, W)
            t[q + "v"] = mat(G * V, W)
            t[q + "q.norm"] = vec(D, 1.0)
            t[q + "k.norm"] = vec(D, 1.0)
            t[q + "sink"] = uni(H, 0.0, 4.0)
            if m.get("v_mix"):
                t[q + "vmix"] = uni(1, 0.2, 0.6)
            t[q + "o"] = mat(W, H * V)
        f = e.get("mlp")
        if f:
            t[p + "norm2"] = vec(W)
            t[p + "mlp.gate"] = mat(f["ff"], W)
            t[p + "mlp.up"] = mat(f["ff"], W)
            t[p + "mlp.down"] = mat(W, f["ff"])
    return t
