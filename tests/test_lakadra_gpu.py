"""The Lakadra decoder against its plain implementation (``plain_lakadra``): every mechanism alone at the level of
its kernel, whole models of several shapes in both precisions, every way of cutting requests into steps and batches
under page pools and state slots that are used again, keys far back, at page edges and at a window's edge in prompts
and in decoding, long decoding through captured steps, and greedy generation through the engine's own entry point.

The models are tiny, with sizes chosen so that nothing is equal by accident: head counts, key, value and latent sizes
differ, a window is no multiple of a page, a layer reads another layer's latent with heads of its own, a layer has no
feed-forward, a router has no groups, no pass-through experts, no shared expert, one choice, a rotation is not
stretched or covers the whole head, a model has no cap and no scale on its logits.  Attention is made sharp through
the score scale, so that a key too many or too few moves the logits far beyond the bounds.
"""
import json
import types

import pytest
import torch

import plain_lakadra as plain

DEV = torch.device("cuda:0")
F64 = torch.float64


# --------------------------------------------------------------------------- model folders

def lightning(heads, dim, vdim, decay):
    return "lightning", {"decay": list(decay), "dim": dim, "heads": heads, "vdim": vdim}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, kv_from=None):
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim, "scale": scale,
             "vdim": vdim, "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return "latent_attention", mixer


def pair(heads, kv_heads, dim, vdim, scale, window, base, dims, factor, width, blocks, conv, left_scale, right_scale):
    left = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim, "rot": {"base": base, "dims": dims}}
    if window:
        left["mask"] = {"size": window}
    if factor:
        left["rot"]["scaling"] = {"factor": factor}
    return "parallel", {"left": left, "right": {"blocks": blocks, "conv": conv, "width": width}, "left_scale": left_scale,
                        "right_scale": right_scale}


def moe(ff, experts, top, identity=0, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity:
        router["identity"] = identity
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"expert": {"ff": ff}, "kind": "moe", "router": router}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": json.loads(json.dumps(mixer[1])), "mlp": mlp}


def configs():
    return {
        # a pair of mixers first: 4 heads on 2 key/value heads of 32 with values of 16, a window of 9 (no multiple of a
        # page), half of each head rotated with positions stretched 4 times; a recurrence of 48 channels in 3 blocks
        # with 3 taps.  Experts in 3 groups of 2 (one of them a pass-through expert), two groups kept, 2 chosen, a shared
        # expert.  Decayed heads of 24 with values of 40; a latent of 40 + 8 rotated; a reader of that latent without
        # feed-forward
        "A": {"architecture": "Lakadra", "vocab": 150, "width": 64, "norm": {"eps": 1e-5}, "logit_scale": 1.5,
              "logit_softcap": 20.0,
              "layers": [layer(pair(4, 2, 32, 16, 0.6, 9, 1000.0, 16, 4.0, 48, 3, 3, 0.8, 1.3), moe(24, 5, 2, 1, (3, 2), 40)),
                         layer(lightning(3, 24, 40, (0.5, 0.9, 0.998)), moe(24, 5, 2, 1, (3, 2), 40)),
                         layer(latent(3, 16, 8, 24, 20, 40, 0.8, 5000.0), moe(16, 3, 1)),
                         layer(lightning(2, 8, 8, (0.97, 0.7)), None),
                         layer(latent(5, 8, 8, 12, 28, 40, 1.1, 5000.0, kv_from=2), None)]},
        # the latent first and its reader last; one decayed head of 136 (more than 128) with values of 8; a pair whose
        # attention sees every key (no mask), rotates whole heads of 64 without stretching and has a key/value head per
        # head (in bfloat16 the tcgen05 prefill kernel), beside a recurrence in one block with 2 taps; a router
        # without groups, pass-through experts or shared expert that chooses one; no scale and no cap on the logits
        "B": {"architecture": "Lakadra", "vocab": 131, "width": 96, "norm": {"eps": 1e-6},
              "layers": [layer(latent(2, 32, 16, 48, 64, 112, 0.7, 300.0), moe(32, 4, 1)),
                         layer(lightning(1, 136, 8, (0.99,)), moe(32, 4, 1)),
                         layer(pair(2, 2, 64, 64, 0.5, None, 20000.0, 64, None, 64, 1, 2, 1.0, 1.0), moe(48, 6, 3, 0, (2, 1))),
                         layer(latent(8, 8, 16, 8, 16, 112, 1.3, 300.0, kv_from=0), moe(32, 4, 2, 2, None, 24))]},
        # two decayed layers in a row; a pair with a window of 3, 3 heads on one key/value head of 48 with values of 80
        # (wider than the keys), a recurrence of 5 blocks of 8 with one tap (no convolution state); 4 experts and 4
        # pass-through experts in 4 groups of which one is kept; a cap without a scale
        "C": {"architecture": "Lakadra", "vocab": 96, "width": 72, "norm": {"eps": 1e-6}, "logit_softcap": 8.0,
              "layers": [layer(lightning(5, 16, 16, (0.3, 0.8, 0.95, 0.99, 0.999)), moe(40, 4, 2, 4, (4, 1), 16)),
                         layer(lightning(2, 40, 24, (0.9, 0.999)), None),
                         layer(pair(3, 1, 48, 80, 0.7, 3, 100.0, 8, 2.0, 40, 5, 1, 1.5, 0.5), moe(40, 4, 2, 4, (4, 1), 16)),
                         layer(latent(3, 8, 24, 32, 24, 24, 0.8, 1.0e6), moe(8, 2, 2))]},
        # pairs only, with heads of the sizes the tcgen05 attention kernels take (64 and 128) under windows of 20 and 40
        # with the unit sink, grouped heads, and a layer without feed-forward between
        "D": {"architecture": "Lakadra", "vocab": 120, "width": 64, "norm": {"eps": 1e-6}, "logit_scale": 0.5,
              "layers": [layer(pair(4, 2, 64, 64, 0.4, 20, 3000.0, 32, 2.0, 32, 2, 4, 1.1, 0.7), moe(16, 3, 2, 1, (2, 1), 24)),
                         layer(pair(2, 1, 128, 128, 0.3, 40, 1.0e5, 128, None, 24, 1, 3, 0.9, 1.2), None),
                         layer(lightning(2, 32, 64, (0.9, 0.99)), moe(16, 3, 2, 1, (2, 1), 24))]},
    }


def write_model(folder, config, seed, edit=None, heat=1.0):
    """Random weights of this test's own making, stored in bfloat16 so that every precision reads the same values.
    ``heat`` scales what sharpens (queries and keys, the experts' squares)."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(torch.bfloat16).contiguous()

    lin = lambda rows, cols, gain=1.0: normal(rows, cols, std=(1.0 + (gain - 1.0) * heat) * cols ** -0.5)  # noqa: E731
    w, width = {}, config["width"]
    w["embed"] = normal(config["vocab"], width, std=0.7)
    for i, entry in enumerate(config["layers"]):
        m, p = entry["mixer"], f"l{i}"
        w[f"{p}.norm1"] = normal(width, std=0.2)
        if entry["type"] == "lightning":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w[f"{p}.mix.q"], w[f"{p}.mix.k"], w[f"{p}.mix.v"] = lin(hd, width, 2.0), lin(hd, width, 2.0), lin(hv, width, 1.5)
            w[f"{p}.mix.g"], w[f"{p}.mix.o"] = lin(hv, width), lin(width, hv, 1.5)
            w[f"{p}.mix.norm"] = normal(hv, std=0.2, mean=1.0)
        elif entry["type"] == "latent_attention":
            h, d, rd, v = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            w[f"{p}.mix.dq"], w[f"{p}.mix.dq.norm"] = lin(m["q_rank"], width), normal(m["q_rank"], std=0.2, mean=1.0)
            w[f"{p}.mix.uq"] = lin(h * (d + rd), m["q_rank"], 1.5)
            if "kv_from" not in m:
                w[f"{p}.mix.dkv"] = lin(m["kv_rank"] + rd, width, 1.5)
                w[f"{p}.mix.dkv.norm"] = normal(m["kv_rank"], std=0.2, mean=1.0)
            w[f"{p}.mix.uk"], w[f"{p}.mix.uv"] = lin(h * d, m["kv_rank"], 1.5), lin(h * v, m["kv_rank"], 1.5)
            w[f"{p}.mix.o"] = lin(width, h * v, 1.5)
        else:
            a, r = m["left"], m["right"]
            h, kv, d, v = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            for role, rows, gain in (("q", h * d, 2.0), ("k", kv * d, 2.0), ("v", kv * v, 1.0)):
                w[f"{p}.mix.left.{role}"], w[f"{p}.mix.left.{role}.b"] = lin(rows, width, gain), normal(rows, std=0.3)
            w[f"{p}.mix.left.g"] = lin(h, width, 2.0)
            w[f"{p}.mix.left.o"], w[f"{p}.mix.left.o.b"] = lin(width, h * v, 1.5), normal(width, std=0.3)
            c, bs = r["width"], r["width"] // r["blocks"]
            for role in ("y", "x"):
                w[f"{p}.mix.right.{role}"], w[f"{p}.mix.right.{role}.b"] = lin(c, width, 1.5), normal(c, std=0.3)
            w[f"{p}.mix.right.conv"], w[f"{p}.mix.right.conv.b"] = normal(c, r["conv"], std=0.5), normal(c, std=0.2)
            for role in ("ra", "ri"):
                w[f"{p}.mix.right.{role}"] = normal(r["blocks"], bs, bs, std=1.5 * bs ** -0.5)
                w[f"{p}.mix.right.{role}.b"] = normal(r["blocks"], bs, std=0.7)
            w[f"{p}.mix.right.lam"] = normal(c, std=1.5, mean=-2.0)  # decays from almost none to fast
            w[f"{p}.mix.right.o"] = lin(width, c, 2.0)
        mlp = entry["mlp"]
        if mlp:
            r = mlp["router"]
            slots = r["experts"] + r.get("identity", 0)
            w[f"{p}.mlp.router"] = lin(slots, width, 3.0)
            w[f"{p}.mlp.correction"] = normal(slots, std=0.15)  # of the order of the scores: it changes choices
            for e in range(r["experts"]):
                w[f"{p}.mlp.e{e}.up"], w[f"{p}.mlp.e{e}.down"] = lin(mlp["expert"]["ff"], width, 1.5), lin(width, mlp["expert"]["ff"])
            if mlp.get("shared"):
                w[f"{p}.mlp.shared.up"], w[f"{p}.mlp.shared.down"] = lin(mlp["shared"]["ff"], width, 1.5), lin(width, mlp["shared"]["ff"])
                w[f"{p}.mlp.shared.sg"] = lin(1, width, 3.0)
    w["final.norm"] = normal(width, std=0.2)
    w["head"] = normal(config["vocab"], width, std=2.0 * width ** -0.5)
    if edit:
        edit(w)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file(w, str(folder / "model.safetensors"))
    return {k: v.to(F64) for k, v in w.items()}


def cooled(config):
    """The same model for the bfloat16 runs: scores less sharp, and a router that chooses every expert it has (no
    groups), since a choice between two experts whose scores are a rounding apart may fall either way in bfloat16 and
    then changes a whole request.  The choice itself is tested in float32 and kernel by kernel."""
    out = json.loads(json.dumps(config))
    for entry in out["layers"]:
        m = entry["mixer"]
        if entry["type"] == "latent_attention":
            m["scale"] = round(m["scale"] * 0.4, 4)
        if entry["type"] == "parallel":
            m["left"]["scale"] = round(m["left"]["scale"] * 0.4, 4)
        if entry["mlp"]:
            r = entry["mlp"]["router"]
            r.pop("groups", None)
            r["top"] = r["experts"] + r.get("identity", 0)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for k, (name, config) in enumerate(configs().items()):
        for suffix, cfg, heat in (("", config, 1.0), ("+", cooled(config), 0.3)):
            folder = tmp_path_factory.mktemp(f"lakadra{name}")
            out[name + suffix] = (str(folder), cfg, write_model(folder, cfg, 900 + k, heat=heat))
    return out


def model_for(models, name, dtype):
    key = name if dtype == "float32" else name + "+"
    return (*models[key], key)


def tokens_of(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


_plain_cache = {}


def plain_logits(name, config, weights, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(config, weights, tokens)
    return _plain_cache[key]


def make_runner(folder, dtype, pages, page=16, seqs=4, graphs=True):
    from slipstream_b200.engine.runner import ModelRunner
    return ModelRunner(folder, dtype=dtype, page_size=page, num_pages=pages, max_num_seqs=seqs, max_model_len=1024,
                       use_cuda_graphs=graphs)


def replay(runner, requests, schedule):
    """``schedule``: steps, each a list of (request, number of tokens).  Logits of every position, per request."""
    from slipstream_b200.engine.runner import StepEntry
    at = {k: 0 for k in requests}
    got = {k: [] for k in requests}
    for step in schedule:
        entries = [StepEntry(k, requests[k][at[k]: at[k] + n], list(range(n))) for k, n in step]
        logits = runner.step(entries).cpu()
        runner.check()
        row = 0
        for k, n in step:
            got[k].append(logits[row: row + n])
            row += n
            at[k] += n
            if at[k] == len(requests[k]):
                runner.release(k)
    runner.cache.check_invariants()
    return {k: torch.cat(v) for k, v in got.items() if v}


def distance(got, want, part=1.0):
    """Root mean square of the difference (means taken off) over that of the plain logits: the worst position, or with
    ``part`` < 1 the position below which that part of all positions lies."""
    d = got.double() - want
    d = d - d.mean(dim=-1, keepdim=True)
    each = d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)
    return float(each.max() if part >= 1.0 else each.quantile(part))


# float32: recurrences of hundreds of steps multiply a rounding of 6e-8 some thousand times; a fault of the kind these
# tests look for (a key, a state, a row off by one) moves the logits by 1e-2 to 1
BOUND = {"float32": 5e-4, "bfloat16": 1e-1}


def close(got, want, dtype):
    if dtype == "float32":
        return distance(got, want) < BOUND[dtype]
    return distance(got, want, 0.9) < BOUND[dtype] and distance(got, want) < 0.5


def step_ctx(q_lens, seq_lens, slots):
    """What the state kernels read of a step: row ranges, positions, lengths after the step and state slots."""
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    positions = [p for n, s in zip(q_lens, seq_lens) for p in range(s - n, s)]
    return types.SimpleNamespace(q_start=as_dev(starts), seq_lens=as_dev(seq_lens), state_slots=as_dev(slots),
                                 positions=as_dev(positions), num_requests=len(q_lens),
                                 is_decode_only=all(n == 1 for n in q_lens))


def in_steps(plan, lens, slots, rows_of, run):
    """Feed each request's rows through ``run(rows of the step, ctx)`` as ``plan`` cuts them; every request's outputs
    in order."""
    at = {k: 0 for k in lens}
    got = {k: [] for k in lens}
    for step in plan:
        ctx = step_ctx([n for _, n in step], [at[k] + n for k, n in step], [slots[k] for k, _ in step])
        out = run(torch.cat([rows_of(k, at[k], at[k] + n) for k, n in step]), ctx)
        row = 0
        for k, n in step:
            got[k].append(out[row: row + n].double().cpu())
            row += n
            at[k] += n
    assert at == lens
    return {k: torch.cat(v) for k, v in got.items()}


PLANS = [  # two requests of 70 and 37 rows: whole; token by token beside portions; portions down to two tokens
    [[("a", 70), ("b", 37)]],
    [[("a", 33)], [("a", 2), ("b", 17)], [("a", 1), ("b", 1)], [("a", 34), ("b", 2)], [("b", 16)], [("b", 1)]],
    [[("b", 37)], [("a", 16)], [("a", 16)], [("a", 3)], [("a", 35)]],
]


def rel(got, want):
    return float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-12))


# --------------------------------------------------------------------------- configuration and structure (no GPU)

def test_configuration_reads_every_branch_and_refuses_what_it_does_not_know():
    from slipstream_b200.config.lakadra_config import LakadraConfig
    from slipstream_b200.config.reader import ConfigError
    from slipstream_b200.registry import resolve_architecture
    c = configs()
    a = LakadraConfig.from_dict(c["A"])
    assert resolve_architecture(c["A"]).name == "Lakadra"
    assert (a.vocab_size, a.hidden_size, a.norm_eps, a.logit_scale, a.logit_softcap) == (150, 64, 1e-5, 1.5, 20.0)
    both, decayed, lat, _, reader = (entry.mixer for entry in a.layers)
    assert (both.left.heads, both.left.kv_heads, both.left.dim, both.left.vdim, both.left.scale, both.left.window) == (4, 2, 32, 16, 0.6, 9)
    assert (both.left.rot.base, both.left.rot.dims, both.left.rot.factor) == (1000.0, 16, 4.0)
    assert (both.right.width, both.right.blocks, both.right.conv, both.left_scale, both.right_scale) == (48, 3, 3, 0.8, 1.3)
    assert (decayed.heads, decayed.dim, decayed.vdim, decayed.decay) == (3, 24, 40, (0.5, 0.9, 0.998))
    assert (lat.heads, lat.dim, lat.rot_dim, lat.vdim, lat.q_rank, lat.kv_rank, lat.scale, lat.kv_from) == (3, 16, 8, 24, 20, 40, 0.8, None)
    assert reader.kv_from == 2 and a.layers[3].mlp is None
    f = a.layers[0].mlp
    assert (f.ff, f.experts, f.top, f.identity, f.group_count, f.group_keep, f.shared_ff) == (24, 5, 2, 1, 3, 2, 40)
    b = LakadraConfig.from_dict(c["B"])
    assert (b.logit_scale, b.logit_softcap) == (1.0, None)
    assert (b.layers[2].mixer.left.window, b.layers[2].mixer.left.rot.factor) == (None, 1.0)
    g = b.layers[0].mlp
    assert (g.identity, g.group_count, g.shared_ff, g.top) == (0, None, None, 1)
    assert LakadraConfig.from_dict(a.to_dict()) == a and LakadraConfig.from_dict(b.to_dict()) == b
    for spoil, text in ((lambda d: d["layers"][0].update(type="attention"), "not a mixer"),
                        (lambda d: d["layers"][0]["mlp"].update(kind="dense"), "kind"),
                        (lambda d: d["layers"][4]["mixer"].update(kv_from=4), "kv_from"),
                        (lambda d: d["layers"][4]["mixer"].update(kv_from=1), "kv_from"),
                        (lambda d: d["layers"][4]["mixer"].update(kv_rank=48), "kv_rank"),
                        (lambda d: d["layers"][1]["mixer"].update(decay=[0.5, 0.9]), "decay"),
                        (lambda d: d["layers"][0]["mixer"]["right"].update(blocks=5), "blocks"),
                        (lambda d: d["layers"][0]["mixer"]["left"].update(kv_heads=3), "kv_heads"),
                        (lambda d: d["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
                        (lambda d: d["layers"][0]["mlp"]["router"].update(top=5), "top"),
                        (lambda d: d.pop("width"), "width")):
        bad = json.loads(json.dumps(c["A"]))
        spoil(bad)
        with pytest.raises(ConfigError, match=text):
            LakadraConfig.from_dict(bad)


def test_model_structure_follows_the_configuration():
    from slipstream_b200.config.lakadra_config import LakadraConfig
    from slipstream_b200.models.lakadra import build_lakadra
    model = build_lakadra(LakadraConfig.from_dict(configs()["A"]))
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["l0.mix.left.q"] == (128, 64) and names["l0.mix.left.k.b"] == (64,) and names["l0.mix.left.v"] == (32, 64)
    assert names["l0.mix.left.g"] == (4, 64) and names["l0.mix.left.o"] == (64, 64) and names["l0.mix.left.o.b"] == (64,)
    assert names["l0.mix.right.ra"] == (3, 16, 16) and names["l0.mix.right.ri.b"] == (3, 16) and names["l0.mix.right.conv"] == (48, 3)
    assert names["l0.mlp.router"] == (6, 64) and names["l0.mlp.correction"] == (6,) and names["l0.mlp.shared.sg"] == (1, 64)
    assert names["l0.mlp.e4.up"] == (24, 64) and "l0.mlp.e5.up" not in names and "l0.mlp.e0.gate" not in names
    assert names["l1.mix.q"] == (72, 64) and names["l1.mix.v"] == (120, 64) and names["l1.mix.norm"] == (120,)
    assert names["l2.mix.dkv"] == (48, 64) and names["l2.mix.uq"] == (72, 20) and "l2.mlp.shared.up" not in names
    assert "l4.mix.dkv" not in names and "l3.mlp.router" not in names and "l0.norm2" not in names
    # two pools of pages: the latent rows (layer 4 reads what layer 2 writes) and the windowed keys of layer 0
    assert [(g.spec.num_kv_heads, g.spec.head_dim, g.spec.window, g.num_entries) for g in model.group_layouts] == [(2, 32, 9, 1), (1, 48, None, 1)]
    assert [[(s.name, tuple(s.shape)) for s in entry] for entry in model.entry_state] == [
        [("right.conv", (2, 48)), ("right.cell", (48,))], [("memory", (3, 24, 40))], [], [("memory", (2, 8, 8))], []]


# --------------------------------------------------------------------------- every mechanism alone

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,dim,vdim", [(3, 24, 40), (1, 136, 8), (2, 5, 33), (4, 64, 64), (1, 256, 70)])
def test_decayed_linear_attention_whole_and_cut_with_slots_used_again(heads, dim, vdim, dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + dim)
    lens, slots = {"a": 70, "b": 37}, {"a": 2, "b": 0}
    width = heads * (2 * dim + 2 * vdim)
    width += -width % 8
    rows = {k: (torch.randn(n, width, generator=g) * 0.8).to(dtype) for k, n in lens.items()}
    decay = torch.tensor([0.999, 0.5, 0.9, 0.97][:heads], dtype=torch.float32)
    weight = torch.randn(heads * vdim, generator=g) * 0.2 + 1.0
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay.tolist()}
    want = {}
    for k, r in rows.items():  # the plain mixer with identity projections: its input is the projected row itself
        x = r.double()
        eye = lambda lo, n: torch.eye(width, dtype=F64)[lo: lo + n]  # noqa: E731
        w = {"p.q": eye(0, heads * dim), "p.k": eye(heads * dim, heads * dim), "p.v": eye(2 * heads * dim, heads * vdim),
             "p.g": eye(heads * (2 * dim + vdim), heads * vdim), "p.norm": weight.double(), "p.o": torch.eye(heads * vdim, dtype=F64)}
        want[k] = plain.lightning(m, w, "p", x, 1e-6)
    for plan in PLANS:
        state = torch.randn(3, heads, dim, vdim, device=DEV)  # what a slot's last owner left
        state[[0, 2]] = 0.0  # the engine clears a slot at admission

        def run(x, ctx):
            x = x.to(DEV)
            mixed = ops.decay_attention(x, decay.to(DEV), state, ctx, heads, dim, vdim)
            g0 = heads * (2 * dim + vdim)
            return ops.gated_rmsnorm(mixed, x[:, g0: g0 + heads * vdim], weight.to(DEV), 1e-6, dtype)

        got = in_steps(plan, lens, slots, lambda k, lo, hi: rows[k][lo:hi], run)
        for k in lens:
            assert rel(got[k], want[k]) < (2e-5 if dtype == torch.float32 else 1.5e-2), (plan, k)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,blocks,taps", [(48, 3, 3), (64, 1, 2), (40, 5, 1), (256, 2, 4), (130, 10, 8)])
def test_gated_linear_recurrence_whole_and_cut(width, blocks, taps, dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(width + taps)
    lens, slots, bs = {"a": 70, "b": 37}, {"a": 1, "b": 2}, width // blocks
    cols = 2 * width + (-2 * width % 8)
    rows = {k: (torch.randn(n, cols, generator=g)).to(dtype) for k, n in lens.items()}
    conv, conv_b = torch.randn(width, taps, generator=g) * 0.5, torch.randn(width, generator=g) * 0.2
    ra, ri = (torch.randn(blocks, bs, bs, generator=g) * 1.5 * bs ** -0.5).to(dtype), (torch.randn(blocks, bs, bs, generator=g) * 1.5 * bs ** -0.5).to(dtype)
    ra_b, ri_b = torch.randn(blocks, bs, generator=g), torch.randn(blocks, bs, generator=g)
    lam = torch.randn(width, generator=g) * 2.0 - 2.0
    want = {}
    for k, r in rows.items():
        eye = torch.eye(cols, dtype=F64)
        w = {"p.y": eye[:width], "p.y.b": torch.zeros(width, dtype=F64), "p.x": eye[width: 2 * width], "p.x.b": torch.zeros(width, dtype=F64),
             "p.conv": conv.double(), "p.conv.b": conv_b.double(), "p.ra": ra.double(), "p.ra.b": ra_b.double(),
             "p.ri": ri.double(), "p.ri.b": ri_b.double(), "p.lam": lam.double(), "p.o": torch.eye(width, dtype=F64)}
        want[k] = plain.gated_linear_recurrence({"width": width, "blocks": blocks}, w, "p", r.double())
    gate_w = torch.cat([ra, ri], dim=1).contiguous().to(DEV)
    gate_b = torch.cat([ra_b, ri_b], dim=1).contiguous().to(DEV)
    for plan in PLANS:
        cell = torch.randn(3, width, device=DEV)
        taps_state = torch.randn(3, taps - 1, width, device=DEV)
        cell[[1, 2]] = 0.0
        taps_state[[1, 2]] = 0.0

        def run(x, ctx):
            x = x.to(DEV)
            u = ops.conv_silu(x, width, width, conv.to(DEV), conv_b.to(DEV), taps_state, ctx, activation=False)
            pre = ops.block_gates(u, gate_w)
            return ops.gated_linear_recurrence(pre, gate_b, u, x[:, :width], lam.to(DEV), 8.0, cell, ctx)

        got = in_steps(plan, lens, slots, lambda k, lo, hi: rows[k][lo:hi], run)
        for k in lens:
            assert rel(got[k], want[k]) < (2e-5 if dtype == torch.float32 else 2.5e-2), (plan, k)


@pytest.mark.gpu
def test_block_gates_of_many_rows_take_the_batched_product_and_agree():
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(5)
    u = torch.randn(300, 96, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(3, 64, 32, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    want = torch.einsum("boi,tbi->bto", w.double().cpu(), u.double().cpu().reshape(300, 3, 32))
    assert rel(ops.block_gates(u, w), want) < 1e-5 and rel(ops.block_gates(u[:100], w), want[:, :100]) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("experts,identity,groups,top", [(5, 1, (3, 2), 2), (4, 0, None, 1), (4, 4, (4, 1), 2), (8, 4, (3, 2), 3),
                                                          (6, 0, (2, 1), 3), (37, 3, (8, 3), 6)])
def test_router_scores_groups_and_choice(experts, identity, groups, top, dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(experts)
    slots, hidden, n = experts + identity, 72, 50
    x = torch.randn(n, hidden, generator=g).to(dtype)
    w = (torch.randn(slots + 1, hidden, generator=g) * 0.4).to(dtype)
    corr = torch.randn(slots, generator=g) * 0.2
    mlp = {"router": {"experts": experts, "top": top, "identity": identity}}
    if groups:
        mlp["router"]["groups"] = {"count": groups[0], "keep": groups[1]}
    ids_want, w_want = plain.route(mlp, {"p.router": w[:slots].double(), "p.correction": corr.double()}, "p", x.double())
    ids, weights, rest = ops.router(x.to(DEV), w.to(DEV), top, softmax=True, correction=corr.to(DEV),
                                    groups=groups[0] if groups else 1, keep=groups[1] if groups else 1, extra=1)
    assert torch.equal(ids.cpu().long(), ids_want), "another choice"
    assert rel(weights, w_want) < 1e-5 and rel(rest[:, 0], x.double() @ w[slots].double()) < 1e-5
    # a correction that lifts a group's weakest expert lifts the group: choices move to it
    lifted = corr.clone()
    lifted[slots - 1] += 5.0
    ids2, weights2 = ops.router(x.to(DEV), w[:slots].contiguous().to(DEV), top, softmax=True, correction=lifted.to(DEV),
                                groups=groups[0] if groups else 1, keep=groups[1] if groups else 1)
    assert bool((ids2[:, 0] == slots - 1).all()) and float(weights2.max()) <= 1.0  # the weight is the score, not the lifted one


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,n,hidden,ff", [(torch.float32, 37, 72, 24), (torch.bfloat16, 37, 72, 24), (torch.bfloat16, 9, 70, 12),
                                               (torch.bfloat16, 300, 64, 40), (torch.bfloat16, 700, 128, 48)])
def test_routed_experts_with_pass_through_and_gated_shared_expert(dtype, n, hidden, ff):
    """All three routes of the grouped products (CUDA cores; mma.sync tiles of 32 and 128 rows; from 1,024 pairs the
    grouped tcgen05 kernel) against the plain sum, expert by expert."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(n)
    experts, identity, top = 5, 3, 2
    x = torch.randn(n, hidden, generator=g).to(dtype)
    up = (torch.randn(experts, ff, hidden, generator=g) * hidden ** -0.5).to(dtype)
    down = (torch.randn(experts, hidden, ff, generator=g) * ff ** -0.5).to(dtype)
    shared = torch.randn(n, hidden, generator=g).to(dtype)
    gate = torch.randn(n, 1, generator=g)
    ids = torch.stack([torch.randperm(experts + identity, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    ids[0] = torch.tensor([experts, experts + 1])  # a token that only hands its input on
    weights = torch.rand(n, top, generator=g)
    want = torch.zeros(n, hidden, dtype=F64)
    for t in range(n):
        for e, s in zip(ids[t].tolist(), weights[t].double()):
            want[t] += s * (plain.expert({"e.up": up[e].double(), "e.down": down[e].double()}, "e", x[t: t + 1].double())[0]
                            if e < experts else x[t].double())
    want += torch.sigmoid(gate.double()) * shared.double()
    y, term_rows = ops.moe_experts_single(x.to(DEV), ids.to(DEV), up.to(DEV), down.to(DEV), experts + identity)
    got = ops.moe_mix(y, term_rows, ids.to(DEV), weights.to(DEV), experts, x.to(DEV), shared.to(DEV), gate.to(DEV))
    assert rel(got, want) < (1e-5 if dtype == torch.float32 else 2e-2)
    from slipstream_b200.ops import check_errors
    check_errors(DEV)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_small_kernels(dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(3)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    x, gates = torch.randn(11, 5 * 24, generator=g).to(dtype), torch.randn(11, 16, generator=g).to(dtype)
    got = x.clone().to(DEV)
    ops.head_gate(got, gates.to(DEV)[:, 3:8], 5, 24)
    want = (x.double().reshape(11, 5, 24) * torch.sigmoid(gates.double()[:, 3:8, None])).reshape(11, 120)
    assert rel(got, want) < tol
    a, b = torch.randn(7, 33, generator=g).to(dtype), torch.randn(7, 33, generator=g).to(dtype)
    assert rel(ops.scaled_sum(a.to(DEV), 1.2, b.to(DEV), -0.7), 1.2 * a.double() - 0.7 * b.double()) < tol
    assert rel(ops.relu_square(a.to(DEV)[:, :32], 20), torch.relu(a.double()[:, :20]) ** 2) < tol
    z = torch.randn(5, 40, generator=g) * 30
    assert rel(ops.soft_cap(z.clone().to(DEV), 12.0, 2.0), 12.0 * torch.tanh(z.double() * 2.0 / 12.0)) < 1e-6
    assert rel(ops.soft_cap(z.clone().to(DEV), None, 0.5), z.double() * 0.5) < 1e-6
    # two branch outputs written into the stream at one point, then the norm with its weight stored around zero
    stream = torch.randn(6, 1, 72, generator=g)
    y1, y2, w = torch.randn(6, 72, generator=g).to(dtype), torch.randn(6, 72, generator=g).to(dtype), torch.randn(72, generator=g) * 0.2
    s = stream.clone().to(DEV)
    one = torch.ones(1, device=DEV)
    got = ops.hc_norm(s, y1.to(DEV), one.reshape(1, 1), one, None, (1.0 + w).to(DEV), 1e-6, dtype, y2=y2.to(DEV))
    total = stream[:, 0].double() + y1.double() + y2.double()
    assert rel(s[:, 0], total) < 1e-6 and rel(got, plain.offset_norm(total, w.double(), 1e-6)) < tol


# --------------------------------------------------------------------------- whole models

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cut_and_batch_gives_the_plain_logits(models, name, dtype):
    """Whole prompts; token by token; portions of several sizes down to two tokens; three unequal requests mixed, in a
    pool smaller than their sum, with two state slots, so that pages and slots are used again."""
    folder, config, weights, key = model_for(models, name, dtype)
    vocab = config["vocab"]
    reqs = {"a": tokens_of(vocab, 70, 1), "b": tokens_of(vocab, 37, 2), "c": tokens_of(vocab, 45, 3)}
    want = {k: plain_logits(key, config, weights, t) for k, t in reqs.items()}
    plans = {
        "whole": [[("a", 70)], [("b", 37)], [("c", 45)]],
        "token by token": [[("b", 1)] for _ in range(37)],
        "portions": [[("a", n)] for n in (16, 1, 2, 13, 3, 2, 17, 16)],
        "mixed": [[("a", 20), ("b", 2)], [("a", 1), ("b", 30)], [("a", 17), ("b", 1)], [("a", 2), ("b", 4)],
                  [("a", 30), ("c", 9)], [("c", 2)], [("c", 34)]],
    }
    for what, plan in plans.items():
        runner = make_runner(folder, dtype, pages=7, seqs=2)  # 112 tokens of cache for up to 115 tokens of requests
        got = replay(runner, reqs, plan)
        for k, logits in got.items():
            assert close(logits, want[k][: logits.shape[0]], dtype), (what, k, distance(logits, want[k][: logits.shape[0]]))


def drawn_config(seed):
    """A model of this design drawn at random: sizes, head counts, the order of the layers, windows, constants and which
    options are present all follow the seed."""
    import random
    rnd = random.Random(seed)
    width = rnd.choice([40, 48, 56, 72, 88, 104, 136])
    n_layers = rnd.randint(3, 6)
    own_latents, layers = [], []
    for i in range(n_layers):
        kind = rnd.choice(["lightning", "latent_attention", "parallel"])
        if kind == "lightning":
            heads = rnd.randint(1, 4)
            mixer = lightning(heads, rnd.randint(3, 72), rnd.randint(3, 72), [round(rnd.uniform(0.3, 0.999), 4) for _ in range(heads)])
        elif kind == "latent_attention":
            if own_latents and rnd.random() < 0.45:
                j = rnd.choice(own_latents)
                src = layers[j]["mixer"]
                mixer = latent(rnd.randint(1, 5), rnd.randint(2, 40), src["rot_dim"], rnd.randint(2, 40), rnd.randint(8, 48), src["kv_rank"],
                               round(rnd.uniform(0.3, 1.0), 3), src["rot"]["base"], kv_from=j)
            else:
                own_latents.append(i)
                mixer = latent(rnd.randint(1, 5), rnd.randint(2, 40), 2 * rnd.randint(1, 10), rnd.randint(2, 40), rnd.randint(8, 48),
                               rnd.randint(8, 60), round(rnd.uniform(0.3, 1.0), 3), rnd.choice([100.0, 10000.0, 5.0e5]))
        else:
            kv = rnd.randint(1, 3)
            dim = 2 * rnd.randint(4, 36)
            blocks = rnd.randint(1, 4)
            mixer = pair(kv * rnd.randint(1, 3), kv, dim, rnd.randint(3, 72), round(rnd.uniform(0.3, 0.9), 3),
                         rnd.choice([None, rnd.randint(2, 45)]), rnd.choice([50.0, 10000.0, 1.0e6]), 2 * rnd.randint(1, dim // 2),
                         rnd.choice([None, 2.0, 8.0]), blocks * rnd.randint(3, 30), blocks, rnd.randint(1, 5),
                         round(rnd.uniform(0.5, 1.5), 2), round(rnd.uniform(0.5, 1.5), 2))
        mlp = None
        if rnd.random() < 0.8:
            experts, identity = rnd.randint(1, 6), rnd.randint(0, 3)
            slots = experts + identity
            groups = None
            counts = [c for c in range(2, slots + 1) if slots % c == 0]
            if counts and rnd.random() < 0.6:
                count = rnd.choice(counts)
                groups = (count, rnd.randint(1, count))
            room = groups[1] * (slots // groups[0]) if groups else slots
            mlp = moe(rnd.randint(4, 40), experts, rnd.randint(1, room), identity, groups, rnd.choice([None, rnd.randint(4, 40)]))
        layers.append(layer(mixer, mlp))
    config = {"architecture": "Lakadra", "vocab": rnd.randint(60, 200), "width": width, "norm": {"eps": rnd.choice([1e-6, 1e-5])},
              "layers": layers}
    if rnd.random() < 0.7:
        config["logit_scale"] = round(rnd.uniform(0.5, 2.5), 2)
    if rnd.random() < 0.7:
        config["logit_softcap"] = round(rnd.uniform(5.0, 40.0), 1)
    return config


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6])
def test_models_drawn_at_random(tmp_path, seed, dtype):
    """Six models whose every size, constant and option follows a seed: whole prompts, and portions beside decoded tokens
    under a pool smaller than the requests with two state slots."""
    from slipstream_b200.config.lakadra_config import LakadraConfig
    config = drawn_config(seed)
    LakadraConfig.from_dict(config)  # the draw is a model the reader takes
    if dtype == "bfloat16":
        config = cooled(config)
    weights = write_model(tmp_path / "m", config, 40 + seed, heat=1.0 if dtype == "float32" else 0.3)
    vocab = config["vocab"]
    reqs = {"a": tokens_of(vocab, 60, seed), "b": tokens_of(vocab, 23, seed + 100), "c": tokens_of(vocab, 41, seed + 200)}
    want = {k: plain.forward(config, weights, t) for k, t in reqs.items()}
    plans = {"whole": [[("a", 60)], [("b", 23)], [("c", 41)]],
             "mixed": [[("a", 19), ("b", 2)], [("a", 1), ("b", 20)], [("a", 38), ("b", 1)], [("a", 2), ("c", 3)], [("c", 1)], [("c", 37)]]}
    for what, plan in plans.items():
        runner = make_runner(str(tmp_path / "m"), dtype, pages=6, seqs=2)
        got = replay(runner, reqs, plan)
        for k, logits in got.items():
            assert close(logits, want[k][: logits.shape[0]], dtype), (seed, what, k, distance(logits, want[k][: logits.shape[0]]))


@pytest.mark.gpu
def test_the_stream_after_every_layer(models):
    from slipstream_b200.engine.context import plan_step, to_device
    from slipstream_b200.engine.runner import StepEntry
    folder, config, weights = models["A"]
    toks = tokens_of(config["vocab"], 40, 9)
    _, want = plain.forward(config, weights, toks, want_layers=True)
    runner = make_runner(folder, "float32", pages=4, seqs=1, graphs=False)
    seen = []

    def tap(pos, stream, pending):
        s = stream.double()
        if pending is not None and hasattr(pending, "y"):  # the layer's two outputs still wait to be added
            s = s + pending.y.double() + (pending.y2.double() if pending.y2 is not None else 0.0)
        seen.append(s.cpu())

    runner.admit("a")
    ctx = to_device(plan_step([StepEntry("a", toks, [39])], runner.cache, runner.config.vocab_size), runner.device)
    ctx.extras["layer_observer"] = tap
    with torch.inference_mode():
        runner.run(ctx)
    runner.check()
    assert len(seen) == len(config["layers"])
    for i, total in enumerate(seen):
        assert float((total - want[i]).abs().max() / want[i].abs().max()) < 2e-5, i


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps_across_windows_and_pages(models, dtype):
    """A prompt of 21 tokens, then 150 tokens one by one (captured decode steps), beside a second request that
    decodes too: every page edge and the window's passing over decoded tokens."""
    folder, config, weights, key = model_for(models, "A", dtype)
    reqs = {"a": tokens_of(config["vocab"], 171, 5), "b": tokens_of(config["vocab"], 160, 6)}
    want = {k: plain_logits(key, config, weights, t) for k, t in reqs.items()}
    plan = [[("a", 21), ("b", 10)]] + [[("a", 1), ("b", 1)] for _ in range(150)]
    runner = make_runner(folder, dtype, pages=24, seqs=2)
    got = replay(runner, reqs, plan)
    for k, logits in got.items():
        assert close(logits, want[k][: logits.shape[0]], dtype), (k, distance(logits, want[k][: logits.shape[0]]))


@pytest.mark.gpu
def test_a_token_far_back_and_keys_at_the_windows_edge_decide(models, tmp_path):
    """What the plain model says about ten tokens some 380 positions back (decayed heads that hardly forget, latent attention
    over every key) and about the keys just inside and just outside a window moves its logits by many times the bound;
    the engine follows in prompts cut at odd places and in decoding.  A window one key too long is far off."""
    folder, config, weights = models["A"]
    vocab = config["vocab"]
    base = tokens_of(vocab, 400, 21)
    other = list(base)
    for i in range(10, 20):  # a run of tokens 380 to 390 positions back
        other[i] = (base[i] + 1) % vocab
    near = list(base)
    near[400 - 9] = (base[400 - 9] + 1) % vocab   # the last key inside the window of the last query
    out = list(base)
    out[400 - 10] = (base[400 - 10] + 1) % vocab  # the first key outside it (it still reaches through other layers)
    plain_all = {k: plain_logits("A", config, weights, t) for k, t in (("base", base), ("other", other), ("near", near), ("out", out))}
    assert distance(plain_all["other"][-1:], plain_all["base"][-1:]) > 20 * BOUND["float32"]
    assert distance(plain_all["near"][-1:], plain_all["base"][-1:]) > 20 * BOUND["float32"]
    plan = [[("x", 100)], [("x", 3)], [("x", 64)], [("x", 201)]] + [[("x", 1)] for _ in range(32)]
    for k, toks in (("base", base), ("other", other), ("near", near), ("out", out)):
        runner = make_runner(folder, "float32", pages=26, seqs=1)
        got = replay(runner, {"x": toks}, plan)["x"]
        assert distance(got, plain_all[k]) < BOUND["float32"], k
    # negative control: the same weights under a window of 10
    wider = json.loads(json.dumps(config))
    wider["layers"][0]["mixer"]["left"]["mask"]["size"] = 10
    (tmp_path / "config.json").write_text(json.dumps(wider))
    import shutil
    shutil.copy(f"{folder}/model.safetensors", tmp_path / "model.safetensors")
    got = replay(make_runner(str(tmp_path), "float32", pages=26, seqs=1), {"x": base}, [[("x", 400)]])["x"]
    assert distance(got, plain_all["base"]) > 20 * BOUND["float32"]


@pytest.mark.gpu
def test_a_state_slot_that_is_not_cleared_shows(models):
    """Negative control: when a slot's last owner's state is left in place, the next request's logits are far off."""
    folder, config, weights = models["C"]
    reqs = {"a": tokens_of(config["vocab"], 30, 1), "b": tokens_of(config["vocab"], 30, 2)}
    want = plain_logits("C", config, weights, reqs["b"])
    runner = make_runner(folder, "float32", pages=8, seqs=1)
    replay(runner, {"a": reqs["a"]}, [[("a", 30)]])
    runner.store.zero_state = lambda slot: None
    got = replay(runner, {"b": reqs["b"]}, [[("b", 30)]])["b"]
    assert distance(got, want) > 20 * BOUND["float32"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D"])
def test_portions_that_take_the_tensor_core_paths(models, name, dtype):
    """600-token portions: the library's batched product for the gates, mma.sync tiles of 128 rows and (from 1,024
    pairs) the grouped tcgen05 kernel for the experts, the tcgen05 prefill attention with a unit sink (model B), and
    with a unit sink under a sliding window (model D)."""
    folder, config, weights, key = model_for(models, name, dtype)
    toks = tokens_of(config["vocab"], 640, 77)
    want = plain_logits(key, config, weights, toks)
    runner = make_runner(folder, dtype, pages=44, seqs=1)
    got = replay(runner, {"x": toks}, [[("x", 600)], [("x", 38)], [("x", 1)], [("x", 1)]])["x"]
    assert close(got, want, dtype), distance(got, want)


@pytest.mark.gpu
def test_greedy_generation_through_the_engine_and_its_scheduler(models):
    """Five prompts of unequal length through `LLMEngine.generate_batch` with prompt portions of 16 tokens and room for
    two requests at a time, so that pages and state slots come back: every generated token is the plain model's
    arg-max (or within a hair of it)."""
    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    for name, dtype, slack in (("A", "float32", 1e-4), ("C+", "bfloat16", 3e-2)):
        folder, config, weights = models[name]
        engine = LLMEngine(EngineConfig.for_model(folder, dtype=dtype, max_model_len=512,
                                                  cache=CacheConfig(block_size=16, num_gpu_blocks=14),
                                                  scheduler=SchedulerConfig(prefill_chunk_size=16, max_num_seqs=2)))
        prompts = [tokens_of(config["vocab"], n, 40 + n) for n in (1, 5, 37, 50, 18)]
        params = SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True)
        outs = engine.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
        for prompt, out in zip(prompts, outs):
            assert len(out) == 12
            toks = list(prompt)
            for tok in out:
                logits = plain.forward(config, weights, toks)[-1]
                assert logits[tok] >= logits.max() - slack * logits.abs().max(), (name, len(toks))
                toks.append(tok)
        assert engine.runner.cache.all_pages_free()
        engine.runner.check()
