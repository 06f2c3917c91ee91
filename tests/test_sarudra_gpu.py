"""The Sarudra decoder against its plain implementation (``plain_sarudra``): every mechanism alone at the level of
its kernel, whole models of several shapes in both precisions, every way of cutting requests into steps and
batches under page pools and state slots that are used again, the edges of windows and pages in prompts and in
decoding, long decoding through captured steps, and greedy generation through the engine's own entry point.

The models are tiny, with sizes chosen so that nothing is equal by accident: head counts, group counts and sizes
that differ between queries, keys, values and state; a rotated part shorter than the head; one, two and three
chosen experts; layers without feed-forward, without mask, without rotation, without shared expert; a state wider
than 128 and heads wider than 128.  Queries and keys pass a weighted norm, so attention is made sharp through the
score scale: one key too many or too few at a window's edge then moves the logits far beyond the bounds.
"""
import json
import types

import pytest
import torch

import plain_sarudra as plain

DEV = torch.device("cuda:0")


# --------------------------------------------------------------------------- model folders

def attention(heads, kv_heads, dim, vdim, scale, rot=None, window=None, softcap=None):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if rot:
        mixer["rot"] = {"dims": rot[0], "base": rot[1]}
    if window:
        mixer["mask"] = {"size": window}
    if softcap:
        mixer["softcap"] = softcap
    return "attention", mixer


def mamba(heads, vdim, state, groups, conv, norm_groups):
    return "mamba2", {"conv": conv, "groups": groups, "heads": heads, "norm_groups": norm_groups, "state": state, "vdim": vdim}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, shared=None):
    out = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return {"type": mixer[0], "mixer": mixer[1], "mlp": mlp}


def configs():
    return {
        # two norm groups; a state-space layer with 3 taps and 3 norm groups over 2 groups of B and C; q/k heads of 24
        # with values of 40 (padded to 48 inside), 16 of 24 elements rotated, a window of 7 (no multiple of a page),
        # two of five experts beside a shared one; a state-space layer without feed-forward; an attention layer
        # without mask, rotation, cap or shared expert, every head with keys of its own
        "P": {"architecture": "Sarudra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5, "groups": 2},
              "embedding": {"scale": 5.0}, "logit_softcap": 12.0,
              "layers": [layer(mamba(4, 12, 20, 2, 3, 3), dense(80)),
                         layer(attention(4, 2, 24, 40, 0.5, (16, 5000.0), window=7, softcap=6.0), moe(5, 2, 24, shared=40)),
                         layer(mamba(6, 8, 12, 3, 2, 1), None),
                         layer(attention(3, 3, 16, 16, 0.6), moe(4, 1, 32))]},
        # one norm group; heads of 64 on one kv head under a window of 40 (the TMA-fed decode kernel with a lower
        # bound on the keys); a state of 130 (more than 128) under heads of 136 (two column tiles), one tap (no
        # convolution state), every head a group of its own; no cap on the logits
        "Q": {"architecture": "Sarudra", "vocab": 131, "width": 128, "norm": {"eps": 1e-6, "groups": 1},
              "embedding": {"scale": 1.0},
              "layers": [layer(attention(8, 1, 64, 64, 0.25, (64, 300000.0), window=40, softcap=30.0), dense(128)),
                         layer(mamba(2, 136, 130, 2, 1, 1), moe(8, 3, 64)),
                         layer(attention(8, 1, 64, 64, 0.25, (32, 100.0), window=16), None)]},
        # heads of 128 under a window of one page and one token; four taps; a state of 64 with one group; eight norm
        # groups; three of six experts with a shared one wider than they are
        "R": {"architecture": "Sarudra", "vocab": 96, "width": 96, "norm": {"eps": 1e-6, "groups": 8},
              "embedding": {"scale": 9.797958971132712}, "logit_softcap": 30.0,
              "layers": [layer(mamba(3, 32, 64, 1, 4, 2), moe(6, 3, 16, shared=48)),
                         layer(attention(2, 1, 128, 128, 0.09, (128, 10000.0), window=17, softcap=50.0), dense(64)),
                         layer(mamba(3, 32, 64, 1, 4, 2), dense(32))]},
    }


def without_close_calls(config):
    """The same model with as many experts as each token chooses.  In bfloat16 a router's choice between two
    experts whose scores are a rounding apart may fall either way, after which a whole request differs; with every
    expert chosen the same kernels run (router, plan, grouped products, each expert weighted by its own score) and
    nothing discrete is left to differ.  The choice itself is tested in float32 and, in bfloat16, kernel by kernel."""
    out = json.loads(json.dumps(config))
    for entry in out["layers"]:
        if entry["mlp"] and entry["mlp"]["kind"] == "moe":
            entry["mlp"]["router"]["experts"] = entry["mlp"]["router"]["top"]
    return out


def write_model(folder, config, seed, dtype=torch.bfloat16):
    """Random weights of this test's own making, stored in bfloat16 so that every precision reads the same values."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype).contiguous()

    def unit(prefix, width, ff):
        w[f"{prefix}.gate"] = normal(ff, width, std=2.0 * width ** -0.5)
        w[f"{prefix}.up"] = normal(ff, width, std=2.0 * width ** -0.5)
        w[f"{prefix}.down"] = normal(width, ff, std=2.0 * ff ** -0.5)

    w, width = {}, config["width"]
    w["embed"] = normal(config["vocab"], width, std=0.3)
    for i, entry in enumerate(config["layers"]):
        m, p = entry["mixer"], f"l{i}"
        w[f"{p}.norm1"] = normal(width, std=0.1, mean=1.0)
        if entry["type"] == "attention":
            w[f"{p}.mix.q"] = normal(m["heads"] * m["dim"], width, std=width ** -0.5)
            w[f"{p}.mix.k"] = normal(m["kv_heads"] * m["dim"], width, std=width ** -0.5)
            w[f"{p}.mix.v"] = normal(m["kv_heads"] * m["vdim"], width, std=2.0 * width ** -0.5)
            w[f"{p}.mix.q.norm"] = normal(m["dim"], std=0.2, mean=1.0)
            w[f"{p}.mix.k.norm"] = normal(m["dim"], std=0.2, mean=1.0)
            w[f"{p}.mix.o"] = normal(width, m["heads"] * m["vdim"], std=2.0 * (m["heads"] * m["vdim"]) ** -0.5)
        else:
            inner, gn = m["heads"] * m["vdim"], m["groups"] * m["state"]
            w[f"{p}.mix.in"] = normal(2 * inner + 2 * gn + m["heads"], width, std=1.5 * width ** -0.5)
            w[f"{p}.mix.conv"] = normal(inner + 2 * gn, m["conv"], std=0.5)
            w[f"{p}.mix.conv.b"] = normal(inner + 2 * gn, std=0.2)
            w[f"{p}.mix.dt_bias"] = normal(m["heads"], std=0.5, mean=-1.0)
            w[f"{p}.mix.A_log"] = normal(m["heads"], std=0.5, mean=-0.5)
            w[f"{p}.mix.D"] = normal(m["heads"], std=0.3, mean=1.0)
            w[f"{p}.mix.norm"] = normal(inner, std=0.1, mean=1.0)
            w[f"{p}.mix.o"] = normal(width, inner, std=2.0 * inner ** -0.5)
        mlp = entry["mlp"]
        if mlp:
            w[f"{p}.norm2"] = normal(width, std=0.1, mean=1.0)
            if mlp["kind"] == "dense":
                unit(f"{p}.mlp", width, mlp["ff"])
            else:
                w[f"{p}.mlp.router"] = normal(mlp["router"]["experts"], width, std=0.1)  # scores far from saturation
                for e in range(mlp["router"]["experts"]):
                    unit(f"{p}.mlp.e{e}", width, mlp["expert"]["ff"])
                if mlp.get("shared"):
                    unit(f"{p}.mlp.shared", width, mlp["shared"]["ff"])
    w["final.norm"] = normal(width, std=0.1, mean=1.0)
    w["head"] = normal(config["vocab"], width, std=2.0 * width ** -0.5)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(config))
    save_file(w, str(folder / "model.safetensors"))
    return w


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for k, (name, config) in enumerate(configs().items()):
        for suffix, cfg in (("", config), ("+", without_close_calls(config))):
            folder = tmp_path_factory.mktemp(f"sarudra{name}")
            out[name + suffix] = (str(folder), cfg, write_model(folder, cfg, 300 + k))
    return out


def model_for(models, name, dtype):
    """(folder, config, weights, key of the plain results): in bfloat16 the variant without close calls."""
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
    return ModelRunner(folder, dtype=dtype, page_size=page, num_pages=pages, max_num_seqs=seqs, max_model_len=4096,
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


def distance(got, want):
    """Root mean square of the difference over that of the plain logits, the worst position."""
    d = got.double() - want
    d = d - d.mean(dim=-1, keepdim=True)
    return float((d.pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)).max())


BOUND = {"float32": 5e-5, "bfloat16": 1e-1}


def step_ctx(q_lens, seq_lens, slots):
    """What the state kernels read of a step: row ranges, lengths after the step and state slots."""
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    as_dev = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)  # noqa: E731
    return types.SimpleNamespace(q_start=as_dev(starts), seq_lens=as_dev(seq_lens), state_slots=as_dev(slots),
                                 num_requests=len(q_lens), is_decode_only=all(n == 1 for n in q_lens))


# --------------------------------------------------------------------------- configuration and structure (no GPU)

def test_configuration_reads_every_branch_and_refuses_what_it_does_not_know():
    from slipstream_b200.config.reader import ConfigError
    from slipstream_b200.config.sarudra_config import SarudraConfig
    from slipstream_b200.registry import resolve_architecture
    c = configs()
    p = SarudraConfig.from_dict(c["P"])
    assert resolve_architecture(c["P"]).name == "Sarudra"
    assert (p.vocab_size, p.hidden_size, p.norm_eps, p.norm_groups, p.embedding_scale, p.logit_softcap) == (200, 64, 1e-5, 2, 5.0, 12.0)
    a, s = p.layers[1].mixer, p.layers[0].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.softcap, a.rot.dims, a.rot.base) == (4, 2, 24, 40, 7, 6.0, 16, 5000.0)
    assert (s.heads, s.vdim, s.state, s.groups, s.conv, s.norm_groups) == (4, 12, 20, 2, 3, 3)
    assert (p.layers[1].mlp.experts, p.layers[1].mlp.top, p.layers[1].mlp.ff, p.layers[1].mlp.shared_ff) == (5, 2, 24, 40)
    last = p.layers[3]
    assert last.mixer.window is None and last.mixer.rot is None and last.mixer.softcap is None and last.mlp.shared_ff is None
    assert p.layers[2].mlp is None and SarudraConfig.from_dict(c["Q"]).logit_softcap is None
    assert SarudraConfig.from_dict(p.to_dict()) == p
    for spoil, text in ((lambda d: d["layers"][0].update(type="recurrent"), "not a mixer"),
                        (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "kind"),
                        (lambda d: d["layers"][1]["mlp"]["router"].update(top=6), "top"),
                        (lambda d: d["layers"][0]["mixer"].update(groups=3), "groups"),
                        (lambda d: d["norm"].update(groups=3), "groups"),
                        (lambda d: d["layers"][1]["mixer"]["rot"].update(dims=26), "rot.dims"),
                        (lambda d: d.pop("vocab"), "vocab")):
        bad = json.loads(json.dumps(c["P"]))
        spoil(bad)
        with pytest.raises(ConfigError, match=text):
            SarudraConfig.from_dict(bad)


def test_model_structure_follows_the_configuration():
    from slipstream_b200.config.sarudra_config import SarudraConfig
    from slipstream_b200.models.sarudra import build_sarudra
    model = build_sarudra(SarudraConfig.from_dict(configs()["P"]))
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["l0.mix.in"] == (2 * 48 + 2 * 40 + 4, 64) and names["l0.mix.conv"] == (48 + 80, 3) and names["l0.mix.conv.b"] == (128,)
    assert names["l1.mix.v"] == (80, 64) and names["l1.mix.o"] == (64, 160) and names["l1.mix.q.norm"] == (24,)
    assert names["l1.mlp.e4.down"] == (64, 24) and names["l1.mlp.shared.gate"] == (40, 64) and names["l1.mlp.router"] == (5, 64)
    assert "l2.norm2" not in names and "l3.mlp.shared.up" not in names and "l1.mlp.e5.up" not in names
    # windowed and unwindowed attention layers keep their pages in pools of their own; state-space layers have none
    assert [(g.spec.head_dim, g.spec.window, g.num_entries) for g in model.group_layouts] == [(48, 7, 1), (16, None, 1)]
    assert [[(s.name, s.shape) for s in entry] for entry in model.entry_state] == [
        [("conv", (2, 128)), ("ssm", (4, 12, 20))], [], [("conv", (1, 120)), ("ssm", (6, 8, 12))], []]


# --------------------------------------------------------------------------- mechanisms alone

@pytest.mark.gpu
@pytest.mark.parametrize("hidden, groups", [(64, 1), (96, 2), (120, 3), (256, 4), (72, 8), (48, 12), (1030, 5)])
def test_grouped_norm_on_a_branch_output(hidden, groups):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(hidden + groups)
    n = 5
    y, stream = torch.randn(n, hidden, generator=g) * 3, torch.randn(n, hidden, generator=g)
    weight, gate = torch.randn(hidden, generator=g), torch.randn(n, hidden + 8, generator=g)
    want = stream.double() + plain.grouped_rms_norm(y.double(), weight.double(), groups, 1e-5)
    dev = stream.to(DEV)
    got = ops.group_norm(y.to(DEV), weight.to(DEV), groups, 1e-5, torch.float32, residual=dev)
    assert torch.allclose(dev.cpu().double(), want, atol=2e-5, rtol=1e-5) and torch.equal(got.cpu(), dev.cpu())
    # the model's last norm: a selection of rows, the stream left alone
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    got = ops.group_norm(stream.to(DEV), weight.to(DEV), groups, 1e-5, torch.float32, rows=rows)
    assert torch.allclose(got.cpu().double(), plain.grouped_rms_norm(stream.double(), weight.double(), groups, 1e-5)[[3, 0]], atol=2e-5)
    # the gate comes before the norm
    gate_dev = gate.to(DEV)[:, 8:]
    got = ops.group_norm(y.to(DEV), weight.to(DEV), groups, 1e-5, torch.float32, gate=gate_dev)
    want = plain.grouped_rms_norm(y.double() * plain.silu(gate[:, 8:].double()), weight.double(), groups, 1e-5)
    assert torch.allclose(got.cpu().double(), want, atol=3e-5, rtol=1e-5)
    # a sum of terms that has not been formed, in bfloat16, added to the stream
    terms, extra = torch.randn(n, 3, hidden, generator=g), torch.randn(n, hidden, generator=g).bfloat16()
    dev = stream.to(DEV)
    got = ops.group_norm(terms.to(DEV), weight.to(DEV), groups, 1e-5, torch.bfloat16, residual=dev, terms=3, extra=extra.to(DEV))
    want = stream.double() + plain.grouped_rms_norm(terms.double().sum(1) + extra.double(), weight.double(), groups, 1e-5)
    assert torch.allclose(dev.cpu().double(), want, atol=3e-5, rtol=1e-5)
    assert torch.equal(got.cpu(), dev.cpu().bfloat16())


@pytest.mark.gpu
@pytest.mark.parametrize("taps, channels", [(4, 70), (3, 300), (2, 16), (1, 40), (8, 33)])
def test_convolution_carries_its_last_inputs_across_steps(taps, channels):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(taps * 100 + channels)
    lens = {"a": 23, "b": 9, "c": 1}
    col0, width = 5, channels + 11
    proj = {k: torch.randn(n, width, generator=g) for k, n in lens.items()}
    w, b = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    want = {k: plain.silu(plain.causal_conv(v[:, col0: col0 + channels].double(), w.double(), b.double())) for k, v in proj.items()}
    state = torch.full((4, taps - 1, channels), 7.0, device=DEV)  # slots as their last owner left them
    slots = {"a": 2, "b": 0, "c": 3}
    for k in slots:
        state[slots[k]].zero_()
    at = {k: 0 for k in lens}
    # portions of one, two and more tokens than taps, alone and side by side; then single tokens together
    plan = [[("a", 5)], [("a", 1), ("b", 2)], [("a", 2), ("b", 6), ("c", 1)], [("a", 9)], [("a", 1), ("b", 1)]] + [[("a", 1)]] * 5
    for step in plan:
        rows = torch.cat([proj[k][at[k]: at[k] + n] for k, n in step]).to(DEV)
        ctx = step_ctx([n for _, n in step], [at[k] + n for k, n in step], [slots[k] for k, _ in step])
        out = ops.conv_silu(rows, col0, channels, w.to(DEV), b.to(DEV), state, ctx).cpu()
        row = 0
        for k, n in step:
            assert torch.allclose(out[row: row + n].double(), want[k][at[k]: at[k] + n], atol=1e-5), (k, at[k], n)
            row += n
            at[k] += n
    assert at == lens and torch.equal(state[1].cpu(), torch.full((taps - 1, channels), 7.0))


@pytest.mark.gpu
@pytest.mark.parametrize("heads, groups, p, n", [(4, 2, 12, 20), (2, 2, 136, 130), (3, 1, 64, 64), (8, 8, 48, 48), (1, 1, 5, 1), (2, 1, 32, 256)])
def test_recurrence_against_the_literal_loop_however_it_is_cut(heads, groups, p, n):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(heads * 1000 + p + n)
    lens, slots = {"a": 37, "b": 6}, {"a": 1, "b": 3}
    inner = heads * p
    xbc = {k: torch.randn(t, inner + 2 * groups * n, generator=g) for k, t in lens.items()}
    dt = {k: torch.randn(t, heads + 3, generator=g) for k, t in lens.items()}
    dt_bias, a_log, d = torch.randn(heads, generator=g) - 1.0, torch.randn(heads, generator=g) * 0.5 - 0.5, torch.randn(heads, generator=g)
    want = {}
    for k, t in lens.items():
        v = xbc[k].double()
        want[k] = plain.state_space_scan(v[:, :inner].reshape(t, heads, p), v[:, inner: inner + groups * n].reshape(t, groups, n),
                                         v[:, inner + groups * n:].reshape(t, groups, n),
                                         plain.softplus(dt[k][:, 3:].double() + dt_bias.double()), a_log.double(), d.double()).reshape(t, inner)
    for plan in ([[("a", 37), ("b", 6)]],
                 [[("a", 16)], [("a", 1), ("b", 2)], [("a", 17), ("b", 1)], [("a", 2), ("b", 3)], [("a", 1)]]):
        state = torch.full((4, heads, p, n), 3.0, device=DEV)
        for s in slots.values():
            state[s].zero_()
        at = {k: 0 for k in lens}
        for step in plan:
            rows = torch.cat([xbc[k][at[k]: at[k] + t] for k, t in step]).to(DEV)
            steps = torch.cat([dt[k][at[k]: at[k] + t] for k, t in step]).to(DEV)
            ctx = step_ctx([t for _, t in step], [at[k] + t for k, t in step], [slots[k] for k, _ in step])
            y = ops.ssm_scan(rows, steps[:, 3:], dt_bias.to(DEV), a_log.to(DEV), d.to(DEV), state, ctx, heads, groups, p, n).cpu()
            row = 0
            for k, t in step:
                assert torch.allclose(y[row: row + t].double(), want[k][at[k]: at[k] + t], atol=2e-4, rtol=1e-4), (k, at[k])
                row += t
                at[k] += t
        assert torch.equal(state[0].cpu(), torch.full((heads, p, n), 3.0))  # a slot nobody holds is left alone


@pytest.mark.gpu
@pytest.mark.parametrize("experts, top, hidden, ff, dtype", [(5, 2, 64, 24, torch.float32), (12, 1, 96, 40, torch.float32),
                                                           (8, 3, 128, 64, torch.bfloat16), (3, 3, 40, 100, torch.float32),
                                                           (70, 4, 72, 16, torch.bfloat16), (3, 2, 64, 72, torch.bfloat16),
                                                           (5, 2, 36, 20, torch.bfloat16)])
def test_router_and_grouped_products(experts, top, hidden, ff, dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(experts * 10 + top)
    n = 150 if experts < 70 else 9
    x = torch.randn(n, hidden, generator=g).to(dtype)
    w = {"r.router": (torch.randn(experts, hidden, generator=g) * 0.2).to(dtype)}
    for e in range(experts):
        w[f"r.e{e}.gate"] = (torch.randn(ff, hidden, generator=g) * hidden ** -0.5).to(dtype)
        w[f"r.e{e}.up"] = (torch.randn(ff, hidden, generator=g) * hidden ** -0.5).to(dtype)
        w[f"r.e{e}.down"] = (torch.randn(hidden, ff, generator=g) * ff ** -0.5).to(dtype)
    ids, scores = ops.router(x.to(DEV), w["r.router"].to(DEV), top)
    logits = x.double() @ w["r.router"].double().T
    want_scores, want_ids = torch.topk(torch.sigmoid(logits), top, dim=-1)
    # a choice may differ from the plain one only where two logits are a rounding apart
    gap = logits.gather(1, want_ids) - logits.gather(1, ids.cpu().long())
    assert float(gap.abs().max()) < 1e-4 * float(logits.abs().max())
    assert torch.allclose(scores.cpu().double(), torch.sigmoid(logits.gather(1, ids.cpu().long())), atol=1e-5)
    gate_up = torch.stack([torch.cat([w[f"r.e{e}.gate"], w[f"r.e{e}.up"]]) for e in range(experts)]).to(DEV)
    down = torch.stack([w[f"r.e{e}.down"] for e in range(experts)]).to(DEV)
    y, term_rows = ops.moe_experts(x.to(DEV), ids, scores, gate_up, down)
    assert term_rows is None
    y = y.cpu().double()
    wd = {k: v.double() for k, v in w.items()}
    worst = 0.0
    for t in range(n):
        for k in range(top):
            e, s = int(ids[t, k]), float(scores[t, k])
            want = plain.gated_unit((s * x[t].double())[None], wd, f"r.e{e}")[0]
            worst = max(worst, float((y[t, k] - want).abs().max() / want.abs().max().clamp_min(1e-3)))
    assert worst < (1e-4 if dtype == torch.float32 else 4e-2)
    combined = ops.moe_combine(y.float().to(DEV), None, dtype).cpu().double()
    assert torch.allclose(combined, y.sum(1).to(dtype).double(), atol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q, n_kv, d, real, vdim, rot_dims, interleaved", [
    (4, 2, 48, 24, 40, 16, False), (3, 1, 64, 64, 64, 64, False), (2, 2, 16, 16, 16, 0, False), (8, 1, 128, 128, 128, 64, False),
    (2, 1, 256, 256, 256, 256, False), (3, 3, 32, 20, 32, 12, True)])
def test_head_norms_rotations_and_page_write(n_q, n_kv, d, real, vdim, rot_dims, interleaved):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(d + n_q + real)
    n, page, pages, base = 9, 4, 7, 777.0
    heads = torch.randn(n, n_q + 2 * n_kv, d, generator=g)
    heads[:, : n_q + n_kv, real:] = 0.0
    heads[:, n_q + n_kv:, vdim:] = 0.0
    rows = torch.cat([heads.reshape(n, -1), torch.randn(n, 24, generator=g)], dim=1)
    positions = torch.tensor([0, 1, 2, 50, 51, 999, 3, 4, 120000], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 20, 21, 0, 13, -1, 27], dtype=torch.int32)
    qw, kw = torch.randn(real, generator=g), torch.randn(real, generator=g)
    f = (base ** (-torch.arange(0, rot_dims, 2, dtype=torch.float64) / max(rot_dims, 1))).float()
    fv = (base ** (-torch.arange(0, vdim, 2, dtype=torch.float64) / vdim)).float()
    kv = torch.zeros(pages, 2, n_kv, page, d)
    dev_rows, dev_kv = rows.to(DEV), kv.to(DEV)
    ops.norm_rope_cache(dev_rows, positions.to(DEV), slots.to(DEV), dev_kv, n_q, n_kv, d, inv_freq=f.to(DEV), rotary_dim=rot_dims,
                        value_inv_freq=fv.to(DEV), value_rotary_dim=vdim, interleaved=interleaved, q_weight=qw.to(DEV),
                        k_weight=kw.to(DEV), norm_dim=real, eps=1e-6)

    def turned(x, dims):
        if dims == 0:
            return x
        if not interleaved:
            return plain.turn_halves(x, positions, dims, base)
        unzip = torch.cat([x[..., 0:dims:2], x[..., 1:dims:2], x[..., dims:]], dim=-1)  # neighbours as halves
        t = plain.turn_halves(unzip, positions, dims, base)
        out = x.clone()
        out[..., 0:dims:2], out[..., 1:dims:2] = t[..., : dims // 2], t[..., dims // 2: dims]
        return out

    q = turned(plain.grouped_rms_norm(heads[:, :n_q, :real].double(), qw.double(), 1, 1e-6), rot_dims)
    k = turned(plain.grouped_rms_norm(heads[:, n_q: n_q + n_kv, :real].double(), kw.double(), 1, 1e-6), rot_dims)
    v = turned(heads[:, n_q + n_kv:, :vdim].double(), vdim)
    out, cache = dev_rows.cpu(), dev_kv.cpu()
    assert torch.equal(out[:, (n_q + 2 * n_kv) * d:], rows[:, (n_q + 2 * n_kv) * d:])
    got_q = out[:, : n_q * d].view(n, n_q, d)
    for t in range(n):
        tol = 3e-5 + 1e-6 * int(positions[t])  # a float32 angle is off by up to 6e-8 of itself
        assert torch.allclose(got_q[t, :, :real].double(), q[t], atol=tol), t
        assert torch.equal(got_q[t, :, real:], torch.zeros(n_q, d - real))
        if int(slots[t]) < 0:
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        assert torch.allclose(cache[pg, 0, :, off, :real].double(), k[t], atol=tol), t
        assert torch.allclose(cache[pg, 1, :, off, :vdim].double(), v[t], atol=tol), t
        assert torch.equal(cache[pg, 1, :, off, vdim:], torch.zeros(n_kv, d - vdim))
    # the turn back: heads' outputs rotated by minus their position
    outs = torch.randn(n, n_q, d, generator=g)
    dev = outs.reshape(n, -1).to(DEV)
    ops.turn_heads(dev, positions.to(DEV), fv.to(DEV), n_q, d, vdim, interleaved=interleaved, sign=-1.0)
    back = dev.cpu().view(n, n_q, d)
    again = turned(back[..., :vdim].double(), vdim)  # turning forward again gives the input
    for t in range(n):
        assert torch.allclose(again[t], outs[t, :, :vdim].double(), atol=3e-5 + 2e-6 * int(positions[t])), t
    assert torch.equal(back[..., vdim:], outs[..., vdim:])


@pytest.mark.gpu
@pytest.mark.parametrize("experts, top, hidden, ff, n", [(4, 2, 128, 128, 600), (6, 3, 64, 192, 400), (3, 1, 256, 64, 1100)])
def test_grouped_products_on_tcgen05(experts, top, hidden, ff, n):
    """Many (token, choice) pairs in bfloat16 with runs of 64 gate and up rows: the grouped two-SM kernel, whose
    outputs stay in sorted order; the norm's kernel and the combining kernel pick them up through the index."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(experts + top + n)
    x = torch.randn(n, hidden, generator=g).bfloat16()
    w = {"r.router": (torch.randn(experts, hidden, generator=g) * 0.2).bfloat16()}
    for e in range(experts):
        w[f"r.e{e}.gate"] = (torch.randn(ff, hidden, generator=g) * hidden ** -0.5).bfloat16()
        w[f"r.e{e}.up"] = (torch.randn(ff, hidden, generator=g) * hidden ** -0.5).bfloat16()
        w[f"r.e{e}.down"] = (torch.randn(hidden, ff, generator=g) * ff ** -0.5).bfloat16()
    ids, scores = ops.router(x.to(DEV), w["r.router"].to(DEV), top)

    def runs(e):  # 64 gate rows, the 64 matching up rows, and so on
        gate, up = w[f"r.e{e}.gate"].reshape(ff // 64, 64, hidden), w[f"r.e{e}.up"].reshape(ff // 64, 64, hidden)
        return torch.stack([gate, up], dim=1).reshape(2 * ff, hidden)

    gate_up = torch.stack([runs(e) for e in range(experts)]).to(DEV)
    down = torch.stack([w[f"r.e{e}.down"] for e in range(experts)]).to(DEV)
    y_sorted, place = ops.moe_experts(x.to(DEV), ids, scores, gate_up, down, run=64)
    ops.check_errors(DEV)
    assert place is not None and y_sorted.dtype == torch.bfloat16 and sorted(place.cpu().tolist()) == list(range(n * top))
    y = y_sorted.cpu().double()[place.cpu().long()].reshape(n, top, hidden)
    wd = {k: v.double() for k, v in w.items()}
    worst = 0.0
    for t in range(0, n, 7):
        for k in range(top):
            e, s = int(ids[t, k]), float(scores[t, k])
            want = plain.gated_unit((s * x[t].double())[None], wd, f"r.e{e}")[0]
            worst = max(worst, float((y[t, k] - want).abs().max() / want.abs().max().clamp_min(1e-3)))
    assert worst < 4e-2
    shared = torch.randn(n, hidden, generator=g).bfloat16()
    combined = ops.moe_combine(y_sorted, shared.to(DEV), torch.bfloat16, place, top).cpu().double()
    assert torch.allclose(combined, (y.sum(1) + shared.double()).bfloat16().double(), atol=1e-6)
    stream, weight = torch.randn(n, hidden, generator=g), torch.randn(hidden, generator=g)
    dev = stream.to(DEV)
    ops.group_norm(y_sorted, weight.to(DEV), 2, 1e-5, torch.bfloat16, residual=dev, terms=top, extra=shared.to(DEV), term_rows=place)
    want = stream.double() + plain.grouped_rms_norm(y.sum(1) + shared.double(), weight.double(), 2, 1e-5)
    assert torch.allclose(dev.cpu().double(), want, atol=3e-5, rtol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q, n_kv, d, rotate_v, normed", [(3, 1, 64, True, True), (8, 2, 128, True, True), (2, 2, 16, False, True),
                                                         (5, 1, 32, True, False), (1, 1, 256, True, True)])
def test_head_kernel_with_sixteen_byte_accesses(n_q, n_kv, d, rotate_v, normed):
    """bfloat16 heads rotated whole: the form of the kernel that takes 8 elements a load, against the plain steps."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(d + n_q)
    n, page, pages, base = 7, 8, 5, 5000.0
    heads = torch.randn(n, n_q + 2 * n_kv, d, generator=g).bfloat16()
    rows = torch.cat([heads.reshape(n, -1), torch.randn(n, 8, generator=g).bfloat16()], dim=1)
    positions = torch.tensor([0, 1, 7, 300, 2, 45, 1000], dtype=torch.int32)
    slots = torch.tensor([3, 4, 39, 8, -1, 17, 0], dtype=torch.int32)
    qw, kw = torch.randn(d, generator=g), torch.randn(d, generator=g)
    f = (base ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).float()
    dev_rows, dev_kv = rows.to(DEV), torch.zeros(pages, 2, n_kv, page, d, dtype=torch.bfloat16, device=DEV)
    ops.norm_rope_cache(dev_rows, positions.to(DEV), slots.to(DEV), dev_kv, n_q, n_kv, d, inv_freq=f.to(DEV), rotary_dim=d,
                        value_inv_freq=f.to(DEV) if rotate_v else None, value_rotary_dim=d if rotate_v else 0,
                        q_weight=qw.to(DEV) if normed else None, k_weight=kw.to(DEV) if normed else None,
                        norm_dim=d if normed else 0, eps=1e-6)
    hd = heads.double()
    q, k, v = hd[:, :n_q], hd[:, n_q: n_q + n_kv], hd[:, n_q + n_kv:]
    if normed:
        q, k = plain.grouped_rms_norm(q, qw.double(), 1, 1e-6), plain.grouped_rms_norm(k, kw.double(), 1, 1e-6)
    q, k = plain.turn_halves(q, positions, d, base), plain.turn_halves(k, positions, d, base)
    if rotate_v:
        v = plain.turn_halves(v, positions, d, base)
    out, cache = dev_rows.cpu(), dev_kv.cpu()
    close = lambda a, b: torch.allclose(a.double(), b, atol=2e-2 * float(b.abs().max()), rtol=1e-2)  # noqa: E731
    assert torch.equal(out[:, (n_q + 2 * n_kv) * d:], rows[:, (n_q + 2 * n_kv) * d:])
    assert close(out[:, : n_q * d].view(n, n_q, d), q)
    for t in range(n):
        if int(slots[t]) < 0:
            assert close(out[t, n_q * d: (n_q + n_kv) * d].view(n_kv, d), k[t])
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        assert close(cache[pg, 0, :, off], k[t]) and close(cache[pg, 1, :, off], v[t]), t


@pytest.mark.gpu
@pytest.mark.parametrize("taps, channels", [(4, 72), (3, 1040), (2, 16), (1, 40)])
def test_convolution_with_sixteen_byte_accesses(taps, channels):
    """bfloat16 rows on 16-byte boundaries: the form that takes 8 channels a thread, across steps and slots."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(taps * 10 + channels)
    lens, slots = {"a": 70, "b": 9}, {"a": 1, "b": 2}
    col0, width = 16, channels + 24
    proj = {k: torch.randn(n, width, generator=g).bfloat16() for k, n in lens.items()}
    w, b = torch.randn(channels, taps, generator=g), torch.randn(channels, generator=g)
    want = {k: plain.silu(plain.causal_conv(v[:, col0: col0 + channels].double(), w.double(), b.double())) for k, v in proj.items()}
    state = torch.zeros((3, taps - 1, channels), device=DEV)
    at = {k: 0 for k in lens}
    for step in [[("a", 35)], [("a", 1), ("b", 2)], [("a", 33), ("b", 6)], [("a", 1), ("b", 1)]]:
        rows = torch.cat([proj[k][at[k]: at[k] + n] for k, n in step]).to(DEV)
        ctx = step_ctx([n for _, n in step], [at[k] + n for k, n in step], [slots[k] for k, _ in step])
        out = ops.conv_silu(rows, col0, channels, w.to(DEV), b.to(DEV), state, ctx).cpu()
        row = 0
        for k, n in step:
            assert torch.allclose(out[row: row + n].double(), want[k][at[k]: at[k] + n], atol=3e-2, rtol=2e-2), (k, at[k], n)
            row += n
            at[k] += n
    assert at == lens and torch.equal(state[0].cpu(), torch.zeros(taps - 1, channels))


@pytest.mark.gpu
def test_soft_cap():
    from slipstream_b200 import ops
    x = torch.linspace(-200, 200, 1001)
    got = ops.soft_cap(x.to(DEV), 15.0).cpu()
    assert torch.allclose(got.double(), plain.soft_cap(x.double(), 15.0), atol=2e-6)


# --------------------------------------------------------------------------- whole models

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
        assert distance(got[k], want[k]) < BOUND[dtype], (k, "whole")
    # token by token
    runner = make_runner(folder, dtype, pages=6, seqs=1)
    got = replay(runner, {"b": reqs["b"]}, [[("b", 1)]] * 41)
    assert distance(got["b"], want["b"]) < BOUND[dtype]
    # portions of changing size, down to two tokens, then single tokens
    cuts = [2, 13, 2, 16, 1, 7, 17, 3] + [1] * 14
    assert sum(cuts) == 75
    got = replay(make_runner(folder, dtype, pages=6, seqs=1), {"a": reqs["a"]}, [[("a", n)] for n in cuts])
    assert distance(got["a"], want["a"]) < BOUND[dtype]
    # unequal requests side by side: portions beside single tokens, requests that end and start in the middle,
    # two state slots and a pool that holds less than all requests
    schedule = [[("a", 30), ("b", 2)], [("a", 1), ("b", 20)], [("a", 1), ("b", 1)], [("a", 20), ("b", 18)],
                [("a", 23), ("c", 1)], [("d", 3), ("e", 19)], [("d", 1), ("e", 1)], [("d", 54)]]
    got = replay(make_runner(folder, dtype, pages=9, seqs=2), reqs, schedule)
    for k in reqs:
        assert distance(got[k], want[k]) < BOUND[dtype], (k, "mixed")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_through_captured_steps(models, dtype):
    """150 single tokens behind a short prompt, two requests side by side: the window passes over decoded tokens and
    page edges many times, the state is carried 150 times, and from the second step on the steps are replayed."""
    folder, config, weights, key = model_for(models, "Q", dtype)
    reqs = {"a": tokens_of(131, 170, 11), "b": tokens_of(131, 153, 12)}
    want = {k: plain_logits(key, config, weights, v) for k, v in reqs.items()}
    runner = make_runner(folder, dtype, pages=12, seqs=2)
    got = replay(runner, reqs, [[("a", 20), ("b", 3)]] + [[("a", 1), ("b", 1)]] * 150)
    for k in reqs:
        assert distance(got[k], want[k]) < BOUND[dtype], k
    assert runner._graphs, "decode steps were not captured"


@pytest.mark.gpu
def test_a_window_off_by_one_or_a_lost_state_would_show(models, tmp_path):
    """Negative controls: the same weights under a window one token longer, and a request whose state slot is not
    cleared, are far outside the bound that the engine meets."""
    from safetensors.torch import save_file
    folder, config, weights = models["Q"]
    toks = tokens_of(131, 90, 21)
    want = plain_logits("Q", config, weights, toks)
    wider = json.loads(json.dumps(config))
    wider["layers"][0]["mixer"]["mask"]["size"] += 1
    (tmp_path / "config.json").write_text(json.dumps(wider))
    save_file(weights, str(tmp_path / "model.safetensors"))
    got = replay(make_runner(str(tmp_path), "float32", pages=8, seqs=1), {"a": toks}, [[("a", 90)]])["a"]
    assert distance(got[:40], want[:40]) < BOUND["float32"]  # inside the window nothing differs
    assert distance(got, want) > 100 * BOUND["float32"]
    runner = make_runner(folder, "float32", pages=8, seqs=1)
    replay(runner, {"x": tokens_of(131, 30, 22)}, [[("x", 30)]])
    runner.reset_state = lambda slot: None  # the next request inherits the slot as it was left
    runner.store.zero_state = lambda slot: None
    got = replay(runner, {"a": toks}, [[("a", 90)]])["a"]
    assert distance(got, want) > 100 * BOUND["float32"]


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_of_one_kind_of_layer_only(tmp_path, dtype):
    """State-space layers alone (no pages at all: the engine runs on state slots only) and attention layers alone
    (no state), cut into portions and decoded."""
    only_state = {"architecture": "Sarudra", "vocab": 90, "width": 64, "norm": {"eps": 1e-6, "groups": 1}, "embedding": {"scale": 2.0},
                  "layers": [layer(mamba(2, 16, 24, 1, 4, 1), dense(64)), layer(mamba(4, 8, 16, 2, 2, 2), None)]}
    only_attention = {"architecture": "Sarudra", "vocab": 90, "width": 64, "norm": {"eps": 1e-6, "groups": 2}, "embedding": {"scale": 2.0},
                      "logit_softcap": 20.0,
                      "layers": [layer(attention(4, 2, 16, 16, 0.5, (16, 1000.0), window=9, softcap=8.0), dense(64)),
                                 layer(attention(2, 1, 32, 32, 0.3, (8, 50.0)), None)]}
    for k, config in enumerate((only_state, only_attention)):
        folder = tmp_path / f"m{k}"
        weights = write_model(folder, config, 500 + k)
        reqs = {"a": tokens_of(90, 45, 41), "b": tokens_of(90, 30, 42)}
        want = {r: plain.logits(config, weights, t) for r, t in reqs.items()}
        schedule = [[("a", 20), ("b", 2)], [("a", 1), ("b", 17)], [("a", 24), ("b", 1)]] + [[("b", 1)]] * 10
        got = replay(make_runner(str(folder), dtype, pages=8, seqs=2), reqs, schedule)
        for r in reqs:
            assert distance(got[r], want[r]) < BOUND[dtype], (k, r)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_portions_at_sizes_the_tensor_core_paths_take(tmp_path, dtype):
    """A wider model whose sizes are in steps of 64: in bfloat16 a portion of 600 tokens with two choices a token is
    1,200 pairs, which the grouped tcgen05 products take; heads of 128 with a window of 200 take the tcgen05 prefill
    attention and the TMA-fed decode kernel; the recurrence takes its cp.async form.  Then portions beside decoded
    tokens, and the window passing over decoded tokens."""
    config = {"architecture": "Sarudra", "vocab": 300, "width": 256, "norm": {"eps": 1e-6, "groups": 4}, "embedding": {"scale": 4.0},
              "logit_softcap": 25.0,
              "layers": [layer(mamba(8, 32, 64, 2, 4, 2), moe(2, 2, 64, shared=128)),
                         layer(attention(4, 2, 128, 128, 0.08, (64, 100000.0), window=200, softcap=25.0), moe(2, 2, 128)),
                         layer(mamba(4, 64, 128, 4, 3, 4), dense(256)),
                         layer(attention(4, 4, 64, 64, 0.12, (64, 10000.0), window=64, softcap=40.0), None)]}
    weights = write_model(tmp_path, config, 77)
    reqs = {"a": tokens_of(300, 700, 51), "b": tokens_of(300, 260, 52)}
    want = {r: plain.logits(config, weights, t) for r, t in reqs.items()}
    schedule = [[("a", 600)], [("a", 70), ("b", 1)], [("a", 1), ("b", 250)]] + [[("a", 1), ("b", 1)]] * 9 + [[("a", 20)]]
    got = replay(make_runner(str(tmp_path), dtype, pages=70, seqs=2), reqs, schedule)
    for r in reqs:
        assert distance(got[r], want[r]) < BOUND[dtype], r


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_token_far_back_is_remembered(tmp_path, dtype):
    """Heads that hardly decay (A_log very low) carry the first token over hundreds of steps, and an unmasked
    attention layer with sharp scores picks single keys far back: two prompts that differ in their first 40 tokens only
    must differ 380 tokens later in the plain implementation, by several times the bound, and the engine must give each
    its own logits, in portions and decoded."""
    from safetensors.torch import save_file
    config = {"architecture": "Sarudra", "vocab": 120, "width": 64, "norm": {"eps": 1e-6, "groups": 2}, "embedding": {"scale": 3.0},
              "layers": [layer(mamba(4, 16, 32, 2, 4, 2), dense(64)),
                         layer(attention(4, 2, 32, 32, 0.45, (32, 10000.0)), None)]}
    weights = write_model(tmp_path, config, 91)
    weights["l0.mix.A_log"] = torch.full((4,), -7.0).bfloat16()  # decay per token about 1 - 1e-3 dt
    save_file(weights, str(tmp_path / "model.safetensors"))
    first = tokens_of(120, 420, 61)
    other = [(t + 17) % 120 for t in first[:40]] + first[40:]
    want = {"a": plain.logits(config, weights, first), "b": plain.logits(config, weights, other)}
    assert distance(want["b"][-20:].float(), want["a"][-20:]) > 3 * BOUND[dtype]  # the first tokens still matter at the end
    reqs = {"a": first, "b": other}
    schedule = [[("a", 300), ("b", 2)], [("a", 100), ("b", 398)]] + [[("a", 1), ("b", 1)]] * 20
    got = replay(make_runner(str(tmp_path), dtype, pages=60, seqs=2), reqs, schedule)
    for r in reqs:
        assert distance(got[r], want[r]) < BOUND[dtype], r


@pytest.mark.gpu
def test_greedy_generation_through_the_engine(models):
    """The package's entry point and scheduler: several requests at once, prompts in portions of 16, pages and state
    slots that come back; every generated token is the plain implementation's arg-max (or within a hair of it)."""
    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    for name, dtype, slack in (("P", "float32", 1e-4), ("Q+", "bfloat16", 3e-2)):
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
