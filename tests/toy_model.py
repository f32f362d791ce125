"""Tiny decoder-shaped module tree whose attribute paths match the names GlowQ's
artefacts use (``model.layers.{L}.self_attn.q_proj`` ...), shared by the golden-vector
generator and the tests.  Only the linears exist; no attention or norms."""
import torch
import torch.nn as nn


class _Attn(nn.Module):
    def __init__(self, hidden, kv, bias):
        super().__init__()
        self.q_proj = nn.Linear(hidden, hidden, bias=bias)
        self.k_proj = nn.Linear(hidden, kv, bias=bias)
        self.v_proj = nn.Linear(hidden, kv, bias=bias)
        self.o_proj = nn.Linear(hidden, hidden, bias=False)


class _Mlp(nn.Module):
    def __init__(self, hidden, inter):
        super().__init__()
        self.gate_proj = nn.Linear(hidden, inter, bias=False)
        self.up_proj = nn.Linear(hidden, inter, bias=False)
        self.down_proj = nn.Linear(inter, hidden, bias=False)


class _Layer(nn.Module):
    def __init__(self, hidden, kv, inter, bias):
        super().__init__()
        self.self_attn = _Attn(hidden, kv, bias)
        self.mlp = _Mlp(hidden, inter)


class _Inner(nn.Module):
    def __init__(self, n_layers, hidden, kv, inter, bias):
        super().__init__()
        self.layers = nn.ModuleList([_Layer(hidden, kv, inter, bias) for _ in range(n_layers)])


class ToyDecoder(nn.Module):
    PROJ = ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj", "self_attn.o_proj",
            "mlp.gate_proj", "mlp.up_proj", "mlp.down_proj")

    def __init__(self, n_layers=2, hidden=256, kv=128, inter=384, bias=False, seed=0):
        super().__init__()
        self.model = _Inner(n_layers, hidden, kv, inter, bias)
        self.lm_head = nn.Linear(hidden, 32, bias=False)
        g = torch.Generator().manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
        self.half()

    def proj(self, layer: int, name: str) -> nn.Module:
        m = self.model.layers[layer]
        for part in name.split("."):
            m = getattr(m, part)
        return m


def make_artifacts(model: ToyDecoder, rank=16, seed=1):
    """Synthetic ``low_rank_shared.pt`` / ``b_ref_map.json`` contents in GlowQ's key scheme
    (src/step2_rsvd.py:487-522): shared B per qkv / mlp group, solo A,B for o_proj, down_proj."""
    g = torch.Generator().manual_seed(seed)
    shared, bmap = {}, {}

    def rnd(*shape):
        return (torch.randn(*shape, generator=g) * 0.01).to(torch.float16)

    for li, layer in enumerate(model.model.layers):
        for gname, members, parent in (("qkv", ("q_proj", "k_proj", "v_proj"), "self_attn"),
                                       ("mlp", ("gate_proj", "up_proj"), "mlp")):
            gk = f"layer{li}_{gname}"
            first = getattr(getattr(layer, parent), members[0])
            shared[f"{gk}.B_shared"] = rnd(rank, first.in_features)
            for m in members:
                lin = getattr(getattr(layer, parent), m)
                shared[f"{gk}.{m}.A"] = rnd(lin.out_features, rank)
                bmap[f"model.layers.{li}.{parent}.{m}.weight"] = f"{gk}.B_shared"
        for parent, m in (("self_attn", "o_proj"), ("mlp", "down_proj")):
            lin = getattr(getattr(layer, parent), m)
            mod = f"model.layers.{li}.{parent}.{m}"
            shared[f"{mod}.A"] = rnd(lin.out_features, rank)
            shared[f"{mod}.B"] = rnd(rank, lin.in_features)
            bmap[f"{mod}.weight"] = f"{mod}.B"
    return shared, bmap
