"""The Bezutar decoder against its plain implementation (``plain_bezutar``): every mechanism alone at the level of
its kernel, whole models of several shapes in both precisions, every way of cutting requests into steps and batches
under page pools and state slots that are used again, keys at page edges and far back in prompts and in decoding,
long decoding through captured steps, and greedy generation through the engine's own entry point.

The models are tiny, with sizes chosen so that nothing is equal by accident: heads, stream and tap counts differ,
query/key sizes differ from value sizes and from the latent's, a layer reads another layer's latent with heads of
its own, a model has one stream (and connection weights all the same), one has the plain residual sum, no pair
table, no position table, no convolution, a rotation without stretching, or a layer without feed-forward.  Attention
is made sharp through the score scale, so that a key too many or too few, or a sink left out, moves the logits far
beyond the bounds.
"""
import json
import math
import types

import pytest
import torch

import plain_bezutar as plain

DEV = torch.device("cuda:0")


# --------------------------------------------------------------------------- model folders

def mlstm(heads, dim, vdim, cap):
    return "mlstm", {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}


def mingru(width):
    return "mingru", {"width": width}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base=None, yarn=None, kv_from=None):
    mixer = {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot_dim": rot_dim, "scale": scale, "vdim": vdim}
    if base:
        mixer["rot"] = {"base": base, "dims": rot_dim}
        if yarn:
            mixer["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return "latent_attention", mixer


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": dict(mixer[1]), "mlp": mlp}


def configs():
    yarn = (6.0, 48, 24.0, 2.0)
    return {
        # three streams, three taps, a pair table of 101 buckets, a position table; a matrix memory of 3 heads of 20
        # with values of 24; latent attention of 3 heads (24 + 8 rotated, values of 20) over a latent of 36 (a cached
        # row of 44 elements, padded to 48), stretched rotation; a recurrence of 90 channels without feed-forward; a
        # layer of 5 heads of 16 that reads the latent of layer 1
        "P": {"architecture": "Bezutar", "vocab": 190, "width": 72, "streams": 3, "norm": {"eps": 1e-5}, "canon": {"taps": 3},
              "embedding": {"bigram": {"buckets": 101, "mul_prev": 31, "mul_cur": 7}}, "max_positions": 1024,
              "layers": [layer(mlstm(3, 20, 24, 10.0), dense(100)),
                         layer(latent(3, 24, 8, 20, 40, 36, 0.9, 5000.0, yarn), dense(88)),
                         layer(mingru(90), None),
                         layer(latent(5, 16, 8, 12, 28, 36, 1.1, 5000.0, yarn, kv_from=1), dense(60))]},
        # the plain residual sum (no streams), no convolution, no pair table, no position table; a rotation that is not
        # stretched; one matrix-memory head of 136 (more than 128) with values of 40; a cached row of 128 elements;
        # the layer that lends its latent is the first, the borrower the last, with other layers between
        "Q": {"architecture": "Bezutar", "vocab": 131, "width": 128, "norm": {"eps": 1e-6},
              "layers": [layer(latent(2, 32, 16, 48, 64, 112, 0.7, 300.0), dense(96)),
                         layer(mingru(300), dense(64)),
                         layer(mlstm(1, 136, 40, 4.0), None),
                         layer(latent(8, 8, 16, 8, 16, 112, 1.3, 300.0, kv_from=0), None)]},
        # one stream with connection weights, five taps, two layers of each recurrent kind in a row, latent attention
        # whose rotated part is wider than the plain one, multipliers that overflow 32 bits when multiplied by a token
        "R": {"architecture": "Bezutar", "vocab": 96, "width": 80, "streams": 1, "norm": {"eps": 1e-6}, "canon": {"taps": 5},
              "embedding": {"bigram": {"buckets": 64, "mul_prev": 2147483647, "mul_cur": 1000003}}, "max_positions": 1024,
              "layers": [layer(mingru(48), dense(72)),
                         layer(mingru(112), None),
                         layer(mlstm(5, 8, 16, 15.0), dense(40)),
                         layer(mlstm(2, 40, 24, 30.0), dense(40)),
                         layer(latent(3, 8, 24, 32, 24, 24, 0.8, 1.0e6, (4.0, 64, 32.0, 1.0)), dense(56))]},
    }


def write_model(folder, config, seed, dtype=torch.bfloat16, edit=None, heat=1.0):
    """Random weights of this test's own making, stored in bfloat16 so that every precision reads the same values.
    ``heat`` scales the weights in front of everything that sharpens (queries, keys, gates of the recurrences, the
    feed-forward's squares): 1 for the float32 runs, lower for the bfloat16 ones (see `cooled`)."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype).contiguous()

    w, width, streams = {}, config["width"], config.get("streams")
    w["embed"] = normal(config["vocab"], width, std=0.7)
    pair = (config.get("embedding") or {}).get("bigram")
    if pair:
        w["bigram"] = normal(pair["buckets"] + 1, width, std=0.5)
    if config.get("max_positions"):
        w["pos"] = normal(config["max_positions"], width, std=0.4)
    for i, entry in enumerate(config["layers"]):
        m, p = entry["mixer"], f"l{i}"
        w[f"{p}.norm1"] = normal(width, std=0.2)
        if config.get("canon"):
            w[f"{p}.canon1"] = normal(width, config["canon"]["taps"], std=0.4)
        for q in (1, 2):
            if streams and (q == 1 or entry["mlp"]):
                w[f"{p}.hc{q}.in"] = normal(streams, std=0.3, mean=1.0 / streams)
                w[f"{p}.hc{q}.out"] = normal(streams, std=0.3, mean=0.7)
                w[f"{p}.hc{q}.mix"] = (torch.eye(streams) * 0.8 + torch.randn(streams, streams, generator=g) * 0.15).to(dtype)
        lin = lambda rows, cols, gain=1.0: normal(rows, cols, std=(1.0 + (gain - 1.0) * heat) * cols ** -0.5)  # noqa: E731
        if entry["type"] == "mlstm":
            hd, hv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            w[f"{p}.mix.q"], w[f"{p}.mix.k"], w[f"{p}.mix.v"] = lin(hd, width, 2.0), lin(hd, width, 2.0), lin(hv, width)
            w[f"{p}.mix.g"], w[f"{p}.mix.o"] = lin(hv, width), lin(width, hv, 2.0)
            w[f"{p}.mix.norm"] = normal(hv, std=0.2, mean=1.0)
            # raw gates of either sign and beyond the cap: the input gate above and below the forget gate's logarithm
            w[f"{p}.mix.i"], w[f"{p}.mix.f"] = lin(m["heads"], width, 3.0), lin(m["heads"], width, 3.0)
            w[f"{p}.mix.i.b"], w[f"{p}.mix.f.b"] = normal(m["heads"], std=1.0, mean=-0.5), normal(m["heads"], std=1.0, mean=2.0)
        elif entry["type"] == "mingru":
            r = m["width"]
            w[f"{p}.mix.z"], w[f"{p}.mix.x"], w[f"{p}.mix.g"] = lin(r, width, 1.5), lin(r, width, 1.5), lin(r, width)
            w[f"{p}.mix.z.b"], w[f"{p}.mix.x.b"] = normal(r, std=0.7, mean=-1.0), normal(r, std=0.5)
            w[f"{p}.mix.o"] = lin(width, r, 2.0)
        else:
            h, d, rd, v = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
            w[f"{p}.mix.dq"], w[f"{p}.mix.dq.norm"] = lin(m["q_rank"], width), normal(m["q_rank"], std=0.2, mean=1.0)
            w[f"{p}.mix.uq"] = lin(h * (d + rd), m["q_rank"], 1.5)
            if "kv_from" not in m:
                w[f"{p}.mix.dkv"] = lin(m["kv_rank"] + rd, width, 1.5)
                w[f"{p}.mix.dkv.norm"] = normal(m["kv_rank"], std=0.2, mean=1.0)
            w[f"{p}.mix.uk"], w[f"{p}.mix.uv"] = lin(h * d, m["kv_rank"], 1.5), lin(h * v, m["kv_rank"], 1.5)
            w[f"{p}.mix.sink"] = normal(h, std=1.0, mean=1.0)
            w[f"{p}.mix.g"], w[f"{p}.mix.o"] = lin(h, width, 2.0), lin(width, h * v, 2.0)
        if entry["mlp"]:
            ff = entry["mlp"]["ff"]
            w[f"{p}.norm2"] = normal(width, std=0.2)
            w[f"{p}.mlp.up"], w[f"{p}.mlp.down"] = lin(ff, width, 1.5), lin(width, ff)
            w[f"{p}.mlp.act"] = normal(2, std=0.6)
    w["final.norm"] = normal(width, std=0.2)
    w["head"] = normal(config["vocab"], width, std=2.0 * width ** -0.5)
    if edit:
        edit(w)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file(w, str(folder / "model.safetensors"))
    return w


def cooled(config):
    """The same model for the bfloat16 runs: scores a third as sharp (the weights are written with ``heat`` 0.3 besides).
    With scores of +-10 the rounding of bfloat16 queries and keys alone moves attention weights by a tenth, and a request's
    logits then differ from the plain ones by more than any bound that would still tell a fault from rounding.  What is
    sharp is tested in float32, where the same code runs; the bfloat16 forms of the kernels are compared one by one."""
    out = json.loads(json.dumps(config))
    for entry in out["layers"]:
        if entry["type"] == "latent_attention":
            entry["mixer"]["scale"] = round(entry["mixer"]["scale"] * 0.35, 4)
    return out


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for k, (name, config) in enumerate(configs().items()):
        for suffix, cfg, heat in (("", config, 1.0), ("+", cooled(config), 0.3)):
            folder = tmp_path_factory.mktemp(f"bezutar{name}")
            out[name + suffix] = (str(folder), cfg, write_model(folder, cfg, 700 + k, heat=heat))
    return out


def model_for(models, name, dtype):
    """(folder, config, weights, key of the plain results): in bfloat16 the cooled variant."""
    key = name if dtype == "float32" else name + "+"
    return (*models[key], key)


def tokens_of(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


_plain_cache = {}


def plain_logits(name, config, weights, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.logits(config, weights, tokens)
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


def close(got, want, dtype):
    """float32: every position within the bound.  bfloat16: the matrix memory divides each head's read-out by its root
    mean square, so a position where a head's read-out nearly cancels multiplies the rounding of q, k and v many times
    over (the plain implementation fed with rounded inputs does the same); nine positions in ten are within the bound
    and none is as far off as unrelated logits would be.  What depends on a token's place is the same code in both
    precisions, and float32 shows it sharply; the bfloat16 forms of the kernels are compared sharply one by one."""
    if dtype == "float32":
        return distance(got, want) < BOUND[dtype]
    return distance(got, want, 0.9) < BOUND[dtype] and distance(got, want) < 0.9


# float32: recurrences of hundreds of steps and heads whose read-out nearly cancels multiply a rounding of 6e-8 some
# thousand times; a fault of the kind these tests look for (a key, a state, a row off by one) moves the logits by 1e-2 to 1
BOUND = {"float32": 5e-4, "bfloat16": 1e-1}


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


def in_steps(plan, lens, slots, rows_of, run, check):
    """Feed each request's rows through ``run(rows of the step, ctx)`` as ``plan`` cuts them, and hand every request's
    part of every step's result to ``check(request, first row, rows)``."""
    at = {k: 0 for k in lens}
    for step in plan:
        ctx = step_ctx([n for _, n in step], [at[k] + n for k, n in step], [slots[k] for k, _ in step])
        out = run([rows_of(k, at[k], at[k] + n) for k, n in step], ctx)
        row = 0
        for k, n in step:
            check(k, at[k], out[row: row + n])
            row += n
            at[k] += n
    assert at == lens


# --------------------------------------------------------------------------- configuration and structure (no GPU)

def test_configuration_reads_every_branch_and_refuses_what_it_does_not_know():
    from slipstream_b200.config.bezutar_config import BezutarConfig
    from slipstream_b200.config.reader import ConfigError
    from slipstream_b200.registry import resolve_architecture
    c = configs()
    p = BezutarConfig.from_dict(c["P"])
    assert resolve_architecture(c["P"]).name == "Bezutar"
    assert (p.vocab_size, p.hidden_size, p.norm_eps, p.streams, p.canon_taps, p.position_rows) == (190, 72, 1e-5, 3, 3, 1024)
    assert (p.pair_hash.buckets, p.pair_hash.mul_prev, p.pair_hash.mul_cur) == (101, 31, 7)
    cell, att, rec, reader = (entry.mixer for entry in p.layers)
    assert (cell.heads, cell.dim, cell.vdim, cell.gate_cap) == (3, 20, 24, 10.0) and rec.width == 90
    assert (att.heads, att.dim, att.rot_dim, att.vdim, att.q_rank, att.kv_rank, att.scale, att.kv_from) == (3, 24, 8, 20, 40, 36, 0.9, None)
    assert (att.rot.base, att.rot.dims, att.rot.scaling) == (5000.0, 8, (6.0, 48, 24.0, 2.0))
    assert reader.kv_from == 1 and p.layers[2].mlp is None and p.layers[3].mlp.ff == 60
    q = BezutarConfig.from_dict(c["Q"])
    assert (q.streams, q.canon_taps, q.pair_hash, q.position_rows) == (None, None, None, None)
    assert q.layers[0].mixer.rot.scaling is None
    assert BezutarConfig.from_dict(p.to_dict()) == p and BezutarConfig.from_dict(q.to_dict()) == q
    for spoil, text in ((lambda d: d["layers"][0].update(type="attention"), "not a mixer"),
                        (lambda d: d["layers"][0]["mlp"].update(kind="moe"), "kind"),
                        (lambda d: d["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                        (lambda d: d["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
                        (lambda d: d["layers"][3]["mixer"].update(kv_rank=40), "kv_rank"),
                        (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=6), "rot.dims"),
                        (lambda d: d["layers"][0]["mixer"].update(gate_cap=0.0), "gate_cap"),
                        (lambda d: d["canon"].update(taps=0), "taps"),
                        (lambda d: d.pop("width"), "width")):
        bad = json.loads(json.dumps(c["P"]))
        spoil(bad)
        with pytest.raises(ConfigError, match=text):
            BezutarConfig.from_dict(bad)


def test_model_structure_follows_the_configuration():
    from slipstream_b200.config.bezutar_config import BezutarConfig
    from slipstream_b200.models.bezutar import build_bezutar
    model = build_bezutar(BezutarConfig.from_dict(configs()["P"]))
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["bigram"] == (102, 72) and names["pos"] == (1024, 72) and names["l0.canon1"] == (72, 3)
    assert names["l0.mix.q"] == (60, 72) and names["l0.mix.v"] == (72, 72) and names["l0.mix.i"] == (3, 72) and names["l0.mix.f.b"] == (3,)
    assert names["l1.mix.dkv"] == (44, 72) and names["l1.mix.uq"] == (96, 40) and names["l1.mix.uv"] == (60, 36) and names["l1.mix.sink"] == (3,)
    assert names["l2.mix.z.b"] == (90,) and names["l2.mix.o"] == (72, 90) and "l2.norm2" not in names and "l2.hc2.in" not in names
    assert names["l3.mix.uk"] == (80, 36) and "l3.mix.dkv" not in names and "l3.mix.dkv.norm" not in names
    assert names["l0.hc1.mix"] == (3, 3) and names["l3.hc2.out"] == (3,) and names["l0.mlp.act"] == (2,)
    # one pool of pages: layer 3 reads the rows layer 1 writes; every layer keeps the last inputs of its convolution
    assert [(g.spec.num_kv_heads, g.spec.head_dim, g.num_entries) for g in model.group_layouts] == [(1, 48, 1)]
    assert [[(s.name, tuple(s.shape)) for s in entry] for entry in model.entry_state] == [
        [("memory", (3, 25, 20)), ("peak", (3,)), ("input_taps", (2, 72))], [("input_taps", (2, 72))],
        [("cell", (90,)), ("input_taps", (2, 72))], [("input_taps", (2, 72))]]
    assert [(s.name, s.dtype) for s in model.embedding_state_specs] == [("last_token", torch.int32)]
    plain_sum = build_bezutar(BezutarConfig.from_dict(configs()["Q"]))
    names = {s.name for s in plain_sum.weight_specs()}
    assert not any(n.split(".")[-2].startswith("hc") for n in names if "." in n) and not {"bigram", "pos", "l0.canon1"} & names
    assert plain_sum.embedding_state_specs == [] and [len(e) for e in plain_sum.entry_state] == [0, 1, 2, 0]


# --------------------------------------------------------------------------- mechanisms alone

CUTS = ([[("a", 37), ("b", 6)]],
        [[("a", 16)], [("a", 1), ("b", 2)], [("a", 17), ("b", 1)], [("a", 2), ("b", 3)], [("a", 1)]],
        [[("a", 2), ("b", 2)]] + [[("a", 1), ("b", 1)]] * 4 + [[("a", 31)]])
# portions that cross the recurrences' batches of 32 and tiles of 128 tokens, cut at, just before and just behind them
LONG_CUTS = ([[("a", 300), ("b", 131)]],
             [[("a", 127), ("b", 1)], [("a", 2), ("b", 129)], [("a", 33), ("b", 1)], [("a", 138)]],
             [[("a", 128)], [("a", 129), ("b", 64)], [("a", 43), ("b", 67)]])
SPANS = {"short": ({"a": 37, "b": 6}, CUTS), "long": ({"a": 300, "b": 131}, LONG_CUTS)}


@pytest.mark.gpu
@pytest.mark.parametrize("buckets, mul_prev, mul_cur, copies, table_dtype",
                         [(101, 31, 7, 3, torch.float32), (64, 2147483647, 1000003, 1, torch.float32), (7, 0, 1, 2, torch.bfloat16),
                          (1, 5, 5, 4, torch.bfloat16)])
def test_embedding_sums_token_pair_and_position_rows(buckets, mul_prev, mul_cur, copies, table_dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(buckets + copies)
    vocab, hidden = 90, 40
    w = {"embed": torch.randn(vocab, hidden, generator=g).to(table_dtype), "bigram": torch.randn(buckets + 1, hidden, generator=g).to(table_dtype),
         "pos": torch.randn(50, hidden, generator=g).to(table_dtype)}
    config = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}}
    lens, slots = {"a": 37, "b": 6}, {"a": 2, "b": 0}
    toks = {k: tokens_of(vocab, n, 3 + n) for k, n in lens.items()}
    want = {k: plain.embed(config, w, t) for k, t in toks.items()}
    dev = {k: v.to(DEV) for k, v in w.items()}
    for plan in CUTS:
        last = torch.full((4,), 55, dtype=torch.int32, device=DEV)  # what the slots' last owners left

        def run(rows, ctx):
            ids = torch.tensor([t for r in rows for t in r], dtype=torch.int32, device=DEV)
            out = ops.embed_sum(ids, dev["embed"], ctx, pair_table=dev["bigram"], pair_hash=(buckets, mul_prev, mul_cur),
                                last_token=last, position_table=dev["pos"], copies=copies).cpu()
            if copies > 1:
                assert all(torch.equal(out[:, 0], out[:, c]) for c in range(1, copies))
                out = out[:, 0]
            return out

        def check(k, at, got):
            assert torch.allclose(got.double(), want[k][at: at + got.shape[0]], atol=1e-5), (k, at)

        in_steps(plan, lens, slots, lambda k, a, b: toks[k][a:b], run, check)
        assert last.cpu().tolist() == [toks["b"][-1], 55, toks["a"][-1], 55]
    # without the two other tables it is the token's row, scaled
    ctx = step_ctx([5], [5], [1])
    ids = torch.tensor(toks["a"][:5], dtype=torch.int32, device=DEV)
    got = ops.embed_sum(ids, dev["embed"], ctx, scale=3.0).cpu()
    assert torch.allclose(got.double(), 3.0 * w["embed"].double()[toks["a"][:5]], atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("taps, channels, dtype", [(3, 72, torch.float32), (5, 80, torch.float32), (1, 40, torch.float32), (2, 33, torch.float32),
                                                   (4, 136, torch.bfloat16), (8, 64, torch.bfloat16)])
def test_convolution_over_a_mixers_input(taps, channels, dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(taps * 100 + channels)
    lens, slots = {"a": 37, "b": 6}, {"a": 1, "b": 3}
    x = {k: torch.randn(n, channels, generator=g).to(dtype) for k, n in lens.items()}
    w = torch.randn(channels, taps, generator=g)
    want = {k: plain.input_convolution(v.double(), w) for k, v in x.items()}
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for plan in CUTS:
        state = torch.full((4, taps - 1, channels), 7.0, device=DEV)
        for s in slots.values():
            state[s].zero_()

        def check(k, at, got):
            assert torch.allclose(got.double(), want[k][at: at + got.shape[0]], atol=tol, rtol=tol), (k, at)

        in_steps(plan, lens, slots, lambda k, a, b: x[k][a:b],
                 lambda rows, ctx: ops.conv_silu(torch.cat(rows).to(DEV), 0, channels, w.to(DEV), None, state, ctx, plus_input=True).cpu(), check)
        assert torch.equal(state[0].cpu(), torch.full((taps - 1, channels), 7.0))  # a slot nobody holds is left alone
        if taps > 1:  # the state ends as the request's last inputs
            assert torch.allclose(state[1].cpu().double(), x["a"][-(taps - 1):].double(), atol=1e-6)


def cell_weights(g, width, heads, dim, vdim, cap):
    lin = lambda rows, cols, gain=1.0: torch.randn(rows, cols, generator=g) * gain * cols ** -0.5  # noqa: E731
    return {"c.q": lin(heads * dim, width, 2.0), "c.k": lin(heads * dim, width, 2.0), "c.v": lin(heads * vdim, width),
            "c.g": lin(heads * vdim, width), "c.o": torch.eye(heads * vdim), "c.norm": torch.randn(heads * vdim, generator=g) * 0.2 + 1.0,
            "c.i": lin(heads, width, cap), "c.f": lin(heads, width, cap), "c.i.b": torch.randn(heads, generator=g) - 0.5,
            "c.f.b": torch.randn(heads, generator=g) + 1.0}


@pytest.mark.gpu
@pytest.mark.parametrize("heads, dim, vdim, cap, dtype", [(3, 20, 24, 10.0, torch.float32), (1, 136, 40, 4.0, torch.float32), (5, 8, 16, 15.0, torch.float32),
                                                        (2, 256, 72, 2.0, torch.float32), (4, 1, 1, 7.0, torch.float32), (2, 64, 128, 15.0, torch.bfloat16),
                                                        (6, 32, 8, 3.0, torch.bfloat16), (2, 44, 30, 6.0, torch.bfloat16)])
@pytest.mark.parametrize("spans", ["short", "long"])
def test_matrix_memory_against_the_literal_loop_however_it_is_cut(heads, dim, vdim, cap, dtype, spans):
    """Raw gates run far beyond the cap on both sides, so that the cap, the running maximum's start at 0 and the lower
    bound exp(-m) of the denominator all take part; the state slots start as their last owners left them.  The literal
    loop reads the projections as the kernel does (rounded to bfloat16 where it runs in bfloat16)."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + dim + vdim)
    width = 48
    (lens, cuts), slots = SPANS[spans], {"a": 1, "b": 3}
    w = cell_weights(g, width, heads, dim, vdim, cap)
    m = {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}
    x = {k: torch.randn(n, width, generator=g) * 1.5 for k, n in lens.items()}
    x["a"][20:] *= 0.05  # tokens that hardly write: |n . q| falls below exp(-m)
    stacked = torch.cat([w["c.q"], w["c.k"], w["c.v"], w["c.g"]]).double()
    gate_rows, gate_bias = torch.cat([w["c.i"], w["c.f"]]).double(), torch.cat([w["c.i.b"], w["c.f.b"]]).double()
    # five more columns behind the four projections, as a padded product leaves them
    proj = {k: torch.cat([v.double() @ stacked.T, torch.ones(v.shape[0], 5, dtype=torch.float64)], dim=1).to(dtype) for k, v in x.items()}
    gates = {k: (v.double() @ gate_rows.T).float() for k, v in x.items()}
    sizes = [heads * dim, heads * dim, heads * vdim, heads * vdim, 5]
    want = {k: _cell_from_projections(*proj[k].double().split(sizes, dim=1)[:4], gates[k].double() + gate_bias, m, w["c.norm"].double(), 1e-5)
            for k in x}
    if dtype == torch.float32:  # and that is the mixer of the design, weights and all
        for k in x:
            assert torch.allclose(want[k], plain.matrix_memory(x[k].double(), w, "c", m, 1e-5), atol=1e-4, rtol=1e-4)
    spread = [float(t) for k in x for t in (gates[k].double() + gate_bias).flatten()]
    assert max(spread) > 1.2 * cap and min(spread) < -1.2 * cap
    tol = 2e-4 if dtype == torch.float32 else 2e-2
    g0 = heads * (2 * dim + vdim)
    for plan in cuts:
        memory = torch.full((4, heads, vdim + 1, dim), 3.0, device=DEV)
        peak = torch.full((4, heads), -2.0, device=DEV)
        for s in slots.values():
            memory[s].zero_()
            peak[s].zero_()

        def run(rows, ctx):
            pr = torch.cat([r[0] for r in rows]).to(DEV)
            ga = torch.cat([r[1] for r in rows]).to(DEV)
            num, nq, peaks = ops.matrix_cell(pr, ga, w["c.i.b"].to(DEV), w["c.f.b"].to(DEV), cap, dim ** -0.5, memory, peak, ctx,
                                             heads, dim, vdim)
            return ops.cell_output(num, nq, peaks, w["c.norm"].to(DEV), pr[:, g0: g0 + heads * vdim], heads, vdim, 1e-5, dtype).cpu()

        def check(k, at, got):
            ref = want[k][at: at + got.shape[0]]
            assert torch.allclose(got.double(), ref, atol=tol, rtol=tol), (k, at, float((got.double() - ref).abs().max()))

        in_steps(plan, lens, slots, lambda k, a, b: (proj[k][a:b], gates[k][a:b]), run, check)
        assert torch.equal(memory[0].cpu(), torch.full((heads, vdim + 1, dim), 3.0)) and torch.equal(peak[2].cpu(), torch.full((heads,), -2.0))


def _cell_from_projections(q, k, v, gate, raw_gates, m, norm_weight, eps):
    """The literal loop of `plain.matrix_memory` behind given projections (identity weights in their place)."""
    heads, dim, vdim = m["heads"], m["dim"], m["vdim"]
    eye = lambda n: torch.eye(n, dtype=torch.float64)  # noqa: E731
    h = torch.cat([q, k, v, gate, raw_gates], dim=1)
    sizes = [heads * dim, heads * dim, heads * vdim, heads * vdim, heads, heads]
    pick, at = {}, 0
    for name, n in zip(("q", "k", "v", "g", "i", "f"), sizes):
        sel = torch.zeros(n, h.shape[1], dtype=torch.float64)
        sel[:, at: at + n] = eye(n)
        pick[f"c.{name}"] = sel
        at += n
    pick.update({"c.i.b": torch.zeros(heads, dtype=torch.float64), "c.f.b": torch.zeros(heads, dtype=torch.float64),
                 "c.norm": norm_weight, "c.o": eye(heads * vdim)})
    return plain.matrix_memory(h, pick, "c", m, eps)


@pytest.mark.gpu
@pytest.mark.parametrize("width, dtype", [(90, torch.float32), (300, torch.float32), (1, torch.float32), (48, torch.bfloat16), (136, torch.bfloat16)])
@pytest.mark.parametrize("spans", ["short", "long"])
def test_gated_recurrence_against_the_literal_loop_however_it_is_cut(width, dtype, spans):
    """Steps of single tokens run the kernel that walks a channel's rows in order; every other step the one that also
    cuts a request's tokens into segments and chains what each segment does to the state in front of it."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(width)
    hidden = 40
    (lens, cuts), slots = SPANS[spans], {"a": 1, "b": 3}
    lin = lambda rows, cols, gain=1.0: torch.randn(rows, cols, generator=g) * gain * cols ** -0.5  # noqa: E731
    w = {"r.z": lin(width, hidden, 2.0), "r.x": lin(width, hidden, 2.0), "r.g": lin(width, hidden), "r.o": torch.eye(width),
         "r.z.b": torch.randn(width, generator=g) - 1.0, "r.x.b": torch.randn(width, generator=g) * 0.5}
    x = {k: torch.randn(n, hidden, generator=g) for k, n in lens.items()}
    stacked = torch.cat([w["r.z"], w["r.x"], w["r.g"]]).double()
    proj = {k: torch.cat([v.double() @ stacked.T, torch.ones(v.shape[0], 3, dtype=torch.float64)], dim=1).to(dtype) for k, v in x.items()}
    # the literal loop behind the projections as the kernel reads them
    pick = {f"r.{n}": torch.cat([torch.zeros(width, i * width), torch.eye(width), torch.zeros(width, (2 - i) * width)], dim=1).double()
            for i, n in enumerate(("z", "x", "g"))}
    bias = torch.cat([w["r.z.b"], w["r.x.b"]])
    want = {}
    for k in x:
        rows = proj[k][:, : 3 * width].double()
        rows[:, : 2 * width] += bias.double()
        want[k] = plain.gated_recurrence(rows, {**pick, "r.z.b": torch.zeros(width), "r.x.b": torch.zeros(width), "r.o": w["r.o"]}, "r", {"width": width})
        if dtype == torch.float32:
            assert torch.allclose(want[k], plain.gated_recurrence(x[k].double(), w, "r", {"width": width}), atol=1e-4, rtol=1e-4)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    for plan in cuts:
        state = torch.full((4, width), 3.0, device=DEV)
        for s in slots.values():
            state[s].zero_()

        def check(k, at, got):
            assert torch.allclose(got.double(), want[k][at: at + got.shape[0]], atol=tol, rtol=tol), (k, at)

        in_steps(plan, lens, slots, lambda k, a, b: proj[k][a:b],
                 lambda rows, ctx: ops.gated_recurrence(torch.cat(rows).to(DEV), width, state, ctx, bias=bias.to(DEV)).cpu(), check)
        assert torch.equal(state[0].cpu(), torch.full((width,), 3.0))


@pytest.mark.gpu
@pytest.mark.parametrize("n, dtype", [(1000, torch.float32), (4096, torch.bfloat16), (1003, torch.bfloat16)])
def test_xielu(n, dtype):
    from slipstream_b200 import ops
    x = torch.linspace(-12.0, 6.0, n).to(dtype)
    for p, q in ((0.3, -0.8), (-2.0, 1.5), (0.0, 0.0)):
        a, b = math.log1p(math.exp(p)), 0.5 + math.log1p(math.exp(q))
        got = ops.xielu(x.clone().to(DEV), a, b).cpu()
        want = plain.xielu(x.double(), torch.tensor(p, dtype=torch.float64), torch.tensor(q, dtype=torch.float64))
        tol = 1e-5 if dtype == torch.float32 else 1e-2
        assert torch.allclose(got.double(), want, atol=tol, rtol=tol)
    # small negative inputs: exp(z) - 1 - z is about z^2 / 2 and must not cancel
    z = torch.tensor([-1e-3, -1e-4, -3e-6, 0.0, 1e-5])
    got = ops.xielu(z.clone().to(DEV), 0.7, 1.2).cpu().double()
    want = plain.xielu(z.double(), torch.tensor(math.log(math.exp(0.7) - 1)).double(), torch.tensor(math.log(math.exp(0.7) - 1)).double())
    assert torch.allclose(got, want, atol=1e-9, rtol=2e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("q_rank, kv_rank, rot_dim, page_dim, yarn, dtype", [(40, 36, 8, 48, (6.0, 48, 24.0, 2.0), torch.float32),
                                                                           (64, 112, 16, 128, None, torch.float32), (24, 24, 24, 48, (4.0, 64, 32.0, 1.0), torch.float32),
                                                                           (16, 8, 2, 16, None, torch.float32), (96, 200, 56, 256, (2.0, 128, 16.0, 1.0), torch.bfloat16)])
def test_latents_are_normed_rotated_and_written_to_their_pages(q_rank, kv_rank, rot_dim, page_dim, yarn, dtype):
    from slipstream_b200 import ops
    from slipstream_b200.parts import RotaryEncoding, YarnRotaryEncoding
    g = torch.Generator().manual_seed(q_rank + kv_rank)
    n, page, pages, base, eps = 9, 4, 8, 700.0, 1e-5
    rot = {"base": base, "dims": rot_dim}
    if yarn:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), yarn))
        enc = YarnRotaryEncoding(rot_dim, base, rot_dim, factor=yarn[0], original=yarn[1], fast=yarn[2], slow=yarn[3])
    else:
        enc = RotaryEncoding(rot_dim, base, rot_dim, exact_table=True)
    from slipstream_b200.parts.base import Runtime
    enc.bind({}, Runtime(DEV, dtype))
    inv_freq, _ = enc.rotary_table()
    want_f, want_scale = plain.rotary_frequencies(rot)
    assert torch.allclose(inv_freq.cpu().double(), want_f, rtol=2e-7) and abs(getattr(enc, "mscale", 1.0) - want_scale) < 1e-7
    down = (torch.randn(n, q_rank + kv_rank + rot_dim + 5, generator=g) * 2.0).to(dtype)
    qw, kw = torch.randn(q_rank, generator=g) * 0.2 + 1.0, torch.randn(kv_rank, generator=g) * 0.2 + 1.0
    positions = torch.tensor([0, 1, 2, 50, 51, 1000, 3, 4, 30000], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 20, 21, 0, 13, -1, 27], dtype=torch.int32)
    kv = torch.full((pages, 2, 1, page, page_dim), 9.0, dtype=dtype, device=DEV)
    cq = ops.latent_rows(down.to(DEV), positions.to(DEV), slots.to(DEV), kv, qw.to(DEV), kw.to(DEV), inv_freq, getattr(enc, "mscale", 1.0),
                         q_rank, kv_rank, rot_dim, eps).cpu()
    d = down.double()
    m = {"kv_rank": kv_rank, "rot": rot}
    w = {"a.dkv": torch.eye(kv_rank + rot_dim, dtype=torch.float64), "a.dkv.norm": kw}
    c, shared = plain.latent_keys(d[:, q_rank: q_rank + kv_rank + rot_dim], w, "a", m, eps, positions)
    tol = 3e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(cq.double(), plain.rms_unit(d[:, :q_rank], eps) * qw.double(), atol=tol, rtol=tol)
    cache = kv.cpu().double()
    for t in range(n):
        if int(slots[t]) < 0:
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        key, value = cache[pg, 0, 0, off], cache[pg, 1, 0, off]
        at = tol + 1e-6 * int(positions[t]) * float(shared[t].abs().max())  # a float32 angle is off by up to 6e-8 of itself
        assert torch.allclose(key[:rot_dim], shared[t], atol=at, rtol=tol), t
        assert torch.allclose(key[rot_dim: rot_dim + kv_rank], c[t], atol=tol, rtol=tol) and torch.allclose(value[:kv_rank], c[t], atol=tol, rtol=tol), t
        assert not key[rot_dim + kv_rank:].any() and not value[kv_rank:].any()
    untouched = [s for s in range(pages * page) if s not in slots.tolist()]
    assert all(bool((cache[s // page, :, 0, s % page] == 9.0).all()) for s in untouched)
    # a layer that reads another layer's rows forms its query latent only
    only = ops.latent_rows(down.to(DEV), positions.to(DEV), None, None, qw.to(DEV), None, inv_freq, 1.0, q_rank, 0, rot_dim, eps).cpu()
    assert torch.equal(only, cq)


@pytest.mark.gpu
@pytest.mark.parametrize("heads, inputs, outputs, turn, dtype", [(3, 24, 36, 8, torch.float32), (5, 16, 36, 8, torch.float32), (2, 32, 112, 16, torch.float32),
                                                               (3, 8, 24, 24, torch.float32), (4, 44, 20, 0, torch.float32), (8, 64, 64, 16, torch.bfloat16),
                                                               (1, 128, 200, 56, torch.bfloat16)])
@pytest.mark.parametrize("n", [7, 150])
def test_products_per_head_with_rotation_and_gate(heads, inputs, outputs, turn, dtype, n):
    """Queries carried into the latent space ([rotated part | product | zeros] per head) and latent-sized outputs
    carried up to values under a gate per head.  With 150 rows the bfloat16 products are the library's batched product
    over strided views, and the kernel only rotates, pads and gates."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(heads * 100 + inputs)
    base = 900.0
    x_head = inputs + turn
    x = torch.randn(n, heads * x_head + 3, generator=g).to(dtype)
    w = (torch.randn(heads, inputs, outputs, generator=g) * inputs ** -0.5).to(dtype)
    positions = torch.tensor(([0, 1, 17, 300, 2, 45, 1000] * 22)[:n], dtype=torch.int32)
    rot = {"base": base, "dims": turn}
    pad = -(-(turn + outputs) // 16) * 16
    out = torch.full((n, heads * pad), 5.0, dtype=dtype, device=DEV)
    f = plain.rotary_frequencies(rot)[0].float() if turn else None
    ops.head_product(x.to(DEV), x_head, w.to(DEV), out, pad, turn=turn, pad_to=pad, positions=positions.to(DEV),
                     inv_freq=f.to(DEV) if turn else None, mscale=1.25)
    heads_in = x[:, : heads * x_head].double().reshape(n, heads, x_head)
    want = torch.einsum("nhi,hio->nho", heads_in[..., :inputs], w.double())
    got = out.cpu().double().reshape(n, heads, pad)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(got[..., turn: turn + outputs], want, atol=tol, rtol=tol) and not got[..., turn + outputs:].any()
    if turn:
        turned = 1.25 * plain.rotate_halves(heads_in[..., inputs:], positions, rot)
        for t in range(n):
            assert torch.allclose(got[t, :, :turn], turned[t], atol=tol + 2e-6 * int(positions[t]), rtol=tol), t
    gates = torch.randn(n, heads + 2, generator=g).to(dtype)
    up = torch.empty((n, heads * outputs), dtype=dtype, device=DEV)
    ops.head_product(x.to(DEV), x_head, w.to(DEV), up, outputs, gates=gates.to(DEV)[:, 1: 1 + heads])
    want = want * torch.sigmoid(gates[:, 1: 1 + heads].double())[:, :, None]
    assert torch.allclose(up.cpu().double().reshape(n, heads, outputs), want, atol=tol, rtol=tol)


# --------------------------------------------------------------------------- whole models

def one_layer(mixer, **keys):
    config = {"architecture": "Bezutar", "vocab": 90, "width": 64, "norm": {"eps": 1e-6}, "layers": [layer(mixer, None)]}
    config.update(keys)
    return config


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_one_mechanism_each(tmp_path, dtype):
    """One layer without feed-forward behind a bare token table, then the same with one more mechanism each: streams,
    the convolution, the pair table, the position table.  Recurrent layers alone run on state slots without any page."""
    att = latent(3, 16, 8, 24, 32, 40, 0.8, 2000.0, (8.0, 32, 16.0, 1.0))
    variants = [one_layer(mlstm(2, 24, 16, 6.0)), one_layer(mingru(72)), one_layer(att),
                one_layer(mingru(72), streams=2), one_layer(att, canon={"taps": 2}),
                one_layer(mlstm(2, 24, 16, 6.0), embedding={"bigram": {"buckets": 37, "mul_prev": 11, "mul_cur": 3}}),
                one_layer(att, max_positions=1024)]
    for k, config in enumerate(variants):
        folder = tmp_path / f"m{k}"
        config = config if dtype == "float32" else cooled(config)
        weights = write_model(folder, config, 800 + k, heat=1.0 if dtype == "float32" else 0.3)
        reqs = {"a": tokens_of(90, 45, 41), "b": tokens_of(90, 30, 42)}
        want = {r: plain.logits(config, weights, t) for r, t in reqs.items()}
        schedule = [[("a", 20), ("b", 2)], [("a", 1), ("b", 17)], [("a", 24), ("b", 1)]] + [[("b", 1)]] * 10
        runner = make_runner(str(folder), dtype, pages=8, seqs=2)
        assert bool(runner.model.group_layouts) == (config["layers"][0]["type"] == "latent_attention")
        got = replay(runner, reqs, schedule)
        for r in reqs:
            assert close(got[r], want[r], dtype), (k, r, distance(got[r], want[r]))


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_the_stream_after_every_layer(models, name):
    """Layer by layer in float32: the sum of the streams behind every layer, as a tap on the model's loop sees it."""
    from slipstream_b200.engine.context import plan_step, to_device
    from slipstream_b200.engine.runner import StepEntry
    folder, config, weights = models[name]
    toks = tokens_of(config["vocab"], 40, 7)
    want, _ = plain.layer_streams(config, weights, toks)
    runner = make_runner(folder, "float32", pages=4, seqs=1, graphs=False)
    seen = []

    def tap(pos, stream, pending):
        s = stream.double()
        s = s if s.dim() == 3 else s[:, None, :]
        if pending is not None and hasattr(pending, "y"):  # the last branch's output still waits to be written
            s = torch.einsum("st,nsw->ntw", pending.mix.double(), s) + pending.out.double()[None, :, None] * pending.y.double()[:, None, :]
        seen.append(s.sum(dim=1).cpu())

    runner.admit("a")
    ctx = to_device(plan_step([StepEntry("a", toks, [39])], runner.cache, runner.config.vocab_size), runner.device)
    ctx.extras["layer_observer"] = tap
    with torch.inference_mode():
        runner.run(ctx)
    runner.check()
    assert len(seen) == len(config["layers"])
    for i, total in enumerate(seen):
        d = float((total - want[i]).abs().max() / want[i].abs().max())
        assert d < 2e-5, (i, d)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_every_way_of_cutting_gives_the_plain_logits(models, name, dtype):
    folder, config, weights, name = model_for(models, name, dtype)
    vocab = config["vocab"]
    reqs = {"a": tokens_of(vocab, 75, 1), "b": tokens_of(vocab, 41, 2), "c": tokens_of(vocab, 1, 3), "d": tokens_of(vocab, 58, 4),
            "e": tokens_of(vocab, 20, 5)}
    want = {k: plain_logits(name, config, weights, v) for k, v in reqs.items()}
    # whole prompts, each alone; pools for one request: pages and slots change hands between them
    runner = make_runner(folder, dtype, pages=6, seqs=1)
    got = replay(runner, reqs, [[(k, len(v))] for k, v in reqs.items()])
    for k in reqs:
        assert close(got[k], want[k], dtype), (k, "whole", distance(got[k], want[k]))
    # token by token
    runner = make_runner(folder, dtype, pages=6, seqs=1)
    got = replay(runner, {"b": reqs["b"]}, [[("b", 1)]] * 41)
    assert close(got["b"], want["b"], dtype)
    # portions of changing size, down to two tokens, then single tokens
    cuts = [2, 13, 2, 16, 1, 7, 17, 3] + [1] * 14
    assert sum(cuts) == 75
    got = replay(make_runner(folder, dtype, pages=6, seqs=1), {"a": reqs["a"]}, [[("a", n)] for n in cuts])
    assert close(got["a"], want["a"], dtype)
    # unequal requests side by side: portions beside single tokens, requests that end and start in the middle,
    # two state slots and a pool that holds less than all requests
    schedule = [[("a", 30), ("b", 2)], [("a", 1), ("b", 20)], [("a", 1), ("b", 1)], [("a", 20), ("b", 18)],
                [("a", 23), ("c", 1)], [("d", 3), ("e", 19)], [("d", 1), ("e", 1)], [("d", 54)]]
    got = replay(make_runner(folder, dtype, pages=9, seqs=2), reqs, schedule)
    for k in reqs:
        assert close(got[k], want[k], dtype), (k, "mixed", distance(got[k], want[k]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(models, dtype):
    """150 single tokens behind a short prompt, two requests side by side: keys cross page edges many times, the states
    are carried 150 times, and from the second step on the steps are replayed."""
    folder, config, weights, key = model_for(models, "P", dtype)
    reqs = {"a": tokens_of(190, 170, 11), "b": tokens_of(190, 153, 12)}
    want = {k: plain_logits(key, config, weights, v) for k, v in reqs.items()}
    runner = make_runner(folder, dtype, pages=24, seqs=2)
    got = replay(runner, reqs, [[("a", 20), ("b", 3)]] + [[("a", 1), ("b", 1)]] * 150)
    for k in reqs:
        assert close(got[k], want[k], dtype), (k, distance(got[k], want[k]))
    assert runner._graphs, "decode steps were not captured"


@pytest.mark.gpu
def test_a_sink_left_out_a_lost_state_or_a_wrong_pair_row_would_show(models, tmp_path):
    """Negative controls: the same weights without sinks, with the running maximum started elsewhere, with a request that
    inherits its slot uncleared, or with another pair row for first tokens, are far outside the bound the engine meets."""
    folder, config, weights = models["P"]
    toks = tokens_of(190, 90, 21)
    want = plain_logits("P", config, weights, toks)
    far = 100 * BOUND["float32"]
    no_sink = {k: (torch.full_like(v, -60.0) if k.endswith(".sink") else v) for k, v in weights.items()}
    assert distance(plain.logits(config, no_sink, toks).float(), want) > far
    one_less = json.loads(json.dumps(config))
    one_less["embedding"]["bigram"]["mul_prev"] += 1
    assert distance(plain.logits(one_less, weights, toks).float(), want) > far
    runner = make_runner(folder, "float32", pages=8, seqs=1)
    replay(runner, {"x": tokens_of(190, 30, 22)}, [[("x", 30)]])
    runner.reset_state = lambda slot: None  # the next request inherits the slot as it was left
    runner.store.zero_state = lambda slot: None
    got = replay(runner, {"a": toks}, [[("a", 90)]])["a"]
    assert distance(got, want) > far
    # the engine itself, for comparison
    got = replay(make_runner(folder, "float32", pages=8, seqs=1), {"a": toks}, [[("a", 90)]])["a"]
    assert distance(got, want) < BOUND["float32"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_at_sizes_the_tensor_core_paths_take(tmp_path, dtype):
    """A wider model whose sizes are in steps of 64: in bfloat16 a portion of 600 tokens takes the tcgen05 products and,
    cached rows being 128 elements, the tcgen05 prefill attention with 8 (and, for the layer that borrows the rows, 4)
    query heads on the one cached row and their sinks; then portions beside decoded tokens."""
    config = {"architecture": "Bezutar", "vocab": 300, "width": 256, "streams": 2, "norm": {"eps": 1e-6}, "canon": {"taps": 4},
              "embedding": {"bigram": {"buckets": 257, "mul_prev": 13, "mul_cur": 5}}, "max_positions": 1024,
              "layers": [layer(mlstm(4, 64, 128, 15.0), dense(512)),
                         layer(latent(8, 64, 64, 64, 192, 64, 0.09, 10000.0, (4.0, 256, 32.0, 1.0)), dense(256)),
                         layer(mingru(384), dense(256)),
                         layer(latent(4, 128, 64, 128, 128, 64, 0.07, 10000.0, (4.0, 256, 32.0, 1.0), kv_from=1), None)]}
    if dtype == "bfloat16":
        config = cooled(config)
    weights = write_model(tmp_path, config, 77, heat=1.0 if dtype == "float32" else 0.3)
    reqs = {"a": tokens_of(300, 700, 51), "b": tokens_of(300, 260, 52)}
    want = {r: plain.logits(config, weights, t) for r, t in reqs.items()}
    schedule = [[("a", 600)], [("a", 70), ("b", 1)], [("a", 1), ("b", 250)]] + [[("a", 1), ("b", 1)]] * 9 + [[("a", 20)]]
    got = replay(make_runner(str(tmp_path), dtype, pages=70, seqs=2), reqs, schedule)
    for r in reqs:
        assert close(got[r], want[r], dtype), (r, distance(got[r], want[r]))


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["mlstm", "mingru", "latent_attention"])
def test_a_token_far_back_is_remembered(tmp_path, dtype, kind):
    """One layer of each kind, made to remember: a matrix memory that hardly forgets (a large forget bias), a recurrence
    whose update gate is nearly shut, attention whose scores are sharp enough to pick single keys among hundreds.  Two
    prompts that differ in their first 40 tokens only must differ 380 tokens later in the plain implementation, far beyond
    the bound, and the engine must give each its own logits, in portions and decoded."""
    mixer = {"mlstm": mlstm(2, 24, 16, 12.0), "mingru": mingru(72), "latent_attention": latent(3, 16, 8, 24, 32, 40, 2.5, 2000.0, (8.0, 32, 16.0, 1.0))}[kind]
    config = one_layer(mixer, canon={"taps": 2})
    config["vocab"] = 120

    def remember(w):
        if kind == "mlstm":
            w["l0.mix.f.b"] = torch.full_like(w["l0.mix.f.b"], 9.0)   # log f about -1e-4: the first tokens stay
            w["l0.mix.f"] = w["l0.mix.f"] * 0.1
        elif kind == "mingru":
            w["l0.mix.z.b"] = torch.full_like(w["l0.mix.z.b"], -6.5)  # z about 1.5e-3 a token
            w["l0.mix.z"] = w["l0.mix.z"] * 0.1

    weights = write_model(tmp_path, config, 91, edit=remember)
    first = tokens_of(120, 420, 61)
    other = [(t + 17) % 120 for t in first[:40]] + first[40:]
    want = {"a": plain.logits(config, weights, first), "b": plain.logits(config, weights, other)}
    # the first tokens still matter at the end: by hundreds of times the bound of the run in float32, which is the sharp one
    assert distance(want["b"][-20:].float(), want["a"][-20:]) > 30 * BOUND["float32"]
    reqs = {"a": first, "b": other}
    schedule = [[("a", 300), ("b", 2)], [("a", 100), ("b", 398)]] + [[("a", 1), ("b", 1)]] * 20
    got = replay(make_runner(str(tmp_path), dtype, pages=60, seqs=2), reqs, schedule)
    for r in reqs:
        assert close(got[r], want[r], dtype), (r, distance(got[r], want[r]))


NEEDLE = 77


def needle_model(folder):
    """One latent-attention layer in which one token's key outweighs every other key for every query: channel 3 of the
    embedding is zero except for the needle token, the shared key part's slowest pair reads that channel alone, and every
    head's query has a large positive element there (read, through the query latent, from a channel that is the same for
    all tokens).  The pair's angle stays below a quarter turn over the prompt, so the score stays large hundreds of
    tokens later."""
    config = one_layer(latent(2, 16, 8, 24, 32, 40, 6.0, 2000.0))

    def edit(w):
        key_channel, same_channel, slow = 3, 11, 8 // 2 - 1
        w["embed"][:, key_channel], w["embed"][:, same_channel] = 0.0, 2.0
        w["embed"][NEEDLE, key_channel] = 8.0
        w["l0.norm1"][key_channel] = w["l0.norm1"][same_channel] = 0.0
        w["l0.mix.dkv"][40:] = 0.0
        w["l0.mix.dkv"][40 + slow, key_channel] = 1.0
        w["l0.mix.dq"][0] = 0.0
        w["l0.mix.dq"][0, same_channel] = 1.0
        for head in range(2):
            w["l0.mix.uq"][head * 24 + 16: (head + 1) * 24] = 0.0
            w["l0.mix.uq"][head * 24 + 16 + slow, 0] = 4.0

    return config, write_model(folder, config, 93, edit=edit)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_one_key_far_back_among_hundreds_decides(tmp_path, dtype):
    """The needle stands at position 5 of 330: with it there every later token attends to it and to little else (not
    even to the sinks); with another token in its place the logits at the end are entirely different.  The engine agrees
    with the plain logits when the needle is many pages back, for a prompt's rows, for portions and for decoded tokens."""
    config, weights = needle_model(tmp_path)
    toks = [t if t != NEEDLE else NEEDLE + 1 for t in tokens_of(90, 330, 71)]
    toks[5] = NEEDLE
    want = plain.logits(config, weights, toks)
    moved = plain.logits(config, weights, toks[:5] + [NEEDLE + 2] + toks[6:])
    assert distance(moved[-30:].float(), want[-30:]) > 0.3
    for schedule in ([[("a", 330)]], [[("a", 300)]] + [[("a", 1)]] * 30, [[("a", 7)], [("a", 250)], [("a", 2)], [("a", 71)]]):
        got = replay(make_runner(str(tmp_path), dtype, pages=24, seqs=1), {"a": toks}, schedule)["a"]
        assert close(got, want, dtype), distance(got, want)


@pytest.mark.gpu
def test_greedy_generation_through_the_engine(models):
    """The package's entry point and scheduler: several requests at once, prompts in portions of 16, pages and state
    slots that come back; every generated token is the plain implementation's arg-max (or within a hair of it)."""
    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    for name, dtype, slack in (("P", "float32", 1e-4), ("R+", "bfloat16", 3e-2)):
        folder, config, weights = models[name]
        engine = LLMEngine(EngineConfig.for_model(folder, dtype=dtype, max_model_len=512,
                                                  cache=CacheConfig(block_size=8, num_gpu_blocks=40),
                                                  scheduler=SchedulerConfig(prefill_chunk_size=16, max_num_seqs=3)))
        prompts = [tokens_of(config["vocab"], n, 20 + n) for n in (1, 9, 37, 50, 23)]
        params = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
        outs = engine.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
        for prompt, out in zip(prompts, outs):
            assert len(out) == 14
            toks = list(prompt)
            for tok in out:
                logits = plain.logits(config, weights, toks)[-1]
                assert logits[tok] >= logits.max() - slack * logits.abs().max(), (name, len(toks))
                toks.append(tok)
        assert engine.runner.cache.all_pages_free()
        engine.runner.check()
