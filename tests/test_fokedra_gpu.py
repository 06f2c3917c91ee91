"""The Fokedra decoder against its plain implementation (``plain_fokedra``): every mechanism alone at the level
of its kernel, whole models of several shapes in both precisions, every way of cutting requests into steps and
batches under page pools that force reuse, edges of chunks and pages in prompts and in decoding, long decoding
through captured steps, and greedy generation through the engine's own entry point and scheduler.

The models are tiny, with sizes chosen so that nothing is equal by accident (query and value heads of different
sizes, a rotated part shorter than the head, three streams, a layer without feed-forward, a layer that reads
another layer's keys under another mask).  Attention is made sharp through the score scale (queries and keys have
unit root mean square, so scaling their projections would change nothing): one key too many or too few at an
edge then moves the logits far beyond the bounds.
"""
import json
import math

import pytest
import torch

import plain_fokedra as plain

DEV = torch.device("cuda:0")


# --------------------------------------------------------------------------- model folders

def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling:
        out["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return out


def layer(heads, kv_heads, dim, vdim, scale, rot_=None, chunk=None, kv_from=None, ff=None, limit=2.0):
    mixer = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if rot_:
        mixer["rot"] = rot_
    if chunk:
        mixer["mask"] = {"size": chunk}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": {"ff": ff, "kind": "dense", "limit": limit} if ff else None}


def configs():
    yarn = (4.0, 64, 8.0, 0.5)
    return {
        # three streams; q/k heads of 24 and values of 40 (padded to 48 inside); 16 of 24 elements rotated, stretched;
        # chunks of 7; a layer without feed-forward that reads layer 0's pages under chunks of 16; a last layer with
        # as many kv heads as heads, no mask and plain frequencies; a feed-forward whose size is no multiple of 64
        "P": {"architecture": "Fokedra", "vocab": 200, "width": 64, "streams": 3, "norm": {"eps": 1e-5},
              "embedding": {"scale": 5.0},
              "layers": [layer(4, 2, 24, 40, 0.6, rot(16, 5000.0, yarn), chunk=7, ff=80, limit=1.0),
                         layer(4, 2, 24, 40, 0.4, rot(16, 5000.0, yarn), chunk=16, kv_from=0),
                         layer(2, 2, 32, 32, 0.5, rot(32, 100.0), ff=96, limit=3.0)]},
        # no streams key (the plain residual sum); heads of 64 on one kv head under chunks of 40 (the TMA-fed decode
        # kernel with a lower bound on the keys); two readers of one layer's pages
        "Q": {"architecture": "Fokedra", "vocab": 131, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
              "layers": [layer(8, 1, 64, 64, 0.3, rot(64, 300000.0, (3.0, 128, 16.0, 1.0)), chunk=40, ff=128),
                         layer(8, 1, 64, 64, 0.3, rot(64, 300000.0, (3.0, 128, 16.0, 1.0)), chunk=40, kv_from=0, ff=64),
                         layer(8, 1, 64, 64, 0.2, rot(64, 300000.0, (3.0, 128, 16.0, 1.0)), kv_from=0, ff=64)]},
        # one stream WITH connection weights; heads of 64 without any mask (the tcgen05 prefill kernel); a layer
        # without rotation; values narrower than keys; chunks of one token and chunks of a page multiple
        "R": {"architecture": "Fokedra", "vocab": 96, "width": 96, "streams": 1, "norm": {"eps": 1e-6},
              "embedding": {"scale": 9.797958971132712},
              "layers": [layer(2, 2, 64, 64, 0.25, rot(32, 1000.0), ff=64),
                         layer(3, 1, 16, 8, 1.0, None, chunk=32, ff=32, limit=0.5),
                         layer(2, 1, 16, 16, 1.0, rot(16, 10.0), chunk=1)]},
        # four streams over a width in steps of 128: in bfloat16 decode steps the o and down products write into the
        # streams themselves; a layer without feed-forward in the middle and at the end of the chain
        "T": {"architecture": "Fokedra", "vocab": 150, "width": 256, "streams": 4, "norm": {"eps": 1e-6},
              "embedding": {"scale": 3.0},
              "layers": [layer(4, 2, 32, 32, 0.4, rot(32, 10000.0, yarn), chunk=24, ff=128),
                         layer(4, 2, 32, 32, 0.4, rot(32, 10000.0, yarn), chunk=24, kv_from=0),
                         layer(4, 4, 32, 32, 0.4, rot(16, 10000.0), ff=256, limit=1.5),
                         layer(8, 1, 32, 32, 0.3, rot(32, 10000.0))]},
        # a width and a vocabulary that are multiples of 8 and of nothing more, keys of 80 elements with values of 16,
        # five heads with kv heads of their own, two streams, chunks that are no multiple of a page
        "U": {"architecture": "Fokedra", "vocab": 1003, "width": 104, "streams": 2, "norm": {"eps": 1e-6},
              "embedding": {"scale": 10.2},
              "layers": [layer(5, 5, 80, 16, 0.2, rot(40, 20000.0, (8.0, 32, 4.0, 2.0)), chunk=50, ff=72, limit=2.0),
                         layer(5, 5, 80, 16, 0.2, rot(40, 20000.0, (8.0, 32, 4.0, 2.0)), chunk=50, kv_from=0, ff=136)]},
    }


def write_model(folder, config, seed, dtype=torch.bfloat16):
    """Random weights of this test's own making, stored in bfloat16 so that every precision reads the same values."""
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(seed)

    def normal(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype).contiguous()

    w, width, s = {}, config["width"], config.get("streams")
    w["embed"] = normal(config["vocab"], width, std=0.3)
    for i, entry in enumerate(config["layers"]):
        m, p = entry["mixer"], f"l{i}"
        w[f"{p}.norm1"] = normal(width, std=0.1, mean=1.0)
        w[f"{p}.mix.q"] = normal(m["heads"] * m["dim"], width, std=width ** -0.5)
        w[f"{p}.mix.g"] = normal(m["heads"] * m["vdim"], width, std=2.0 * width ** -0.5)
        w[f"{p}.mix.o"] = normal(width, m["heads"] * m["vdim"], std=2.0 * (m["heads"] * m["vdim"]) ** -0.5)
        if "kv_from" not in m:
            w[f"{p}.mix.k"] = normal(m["kv_heads"] * m["dim"], width, std=width ** -0.5)
            w[f"{p}.mix.v"] = normal(m["kv_heads"] * m["vdim"], width, std=2.0 * width ** -0.5)
        subs = [1]
        if entry["mlp"]:
            ff = entry["mlp"]["ff"]
            w[f"{p}.norm2"] = normal(width, std=0.1, mean=1.0)
            w[f"{p}.mlp.gate"] = normal(ff, width, std=2.0 * width ** -0.5)
            w[f"{p}.mlp.up"] = normal(ff, width, std=2.0 * width ** -0.5)
            w[f"{p}.mlp.down"] = normal(width, ff, std=2.0 * ff ** -0.5)
            subs.append(2)
        if s:
            for q in subs:
                w[f"{p}.hc{q}.in"] = normal(s, std=0.3, mean=0.7)
                w[f"{p}.hc{q}.out"] = normal(s, std=0.4, mean=0.8)
                w[f"{p}.hc{q}.mix"] = (torch.eye(s) * 0.7 + torch.randn(s, s, generator=g) * 0.3).to(dtype).contiguous()
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
        folder = tmp_path_factory.mktemp(f"fokedra{name}")
        out[name] = (str(folder), config, write_model(folder, config, 100 + k))
    return out


def tokens_of(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return [int(t) for t in torch.randint(0, vocab, (n,), generator=g)]


_plain_cache = {}


def plain_logits(name, config, weights, tokens):
    key = (name, tuple(tokens))
    if key not in _plain_cache:
        _plain_cache[key] = plain.forward(config, weights, tokens)[0]
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


# float32 measures 3e-6 to 7e-6 on these models and bfloat16 3e-2 to 6e-2 (sharp attention over widths of 64 to 128);
# one key too many at a chunk's edge measures above 0.8 (`test_a_key_that_should_not_be_seen_would_show`)
BOUND = {"float32": 5e-5, "bfloat16": 1e-1}


# --------------------------------------------------------------------------- configuration and tables (no GPU)

def test_configuration_reads_every_branch_and_refuses_what_it_does_not_know():
    from slipstream_b200.config.fokedra_config import FokedraConfig
    from slipstream_b200.config.reader import ConfigError
    from slipstream_b200.registry import resolve_architecture
    c = configs()
    p = FokedraConfig.from_dict(c["P"])
    assert resolve_architecture(c["P"]).name == "Fokedra"
    assert (p.vocab_size, p.hidden_size, p.streams, p.norm_eps, p.embedding_scale) == (200, 64, 3, 1e-5, 5.0)
    assert p.layers[0].mixer.rot.scaling == (4.0, 64.0, 8.0, 0.5) and p.layers[0].mixer.chunk == 7
    assert p.layers[1].mixer.kv_from == 0 and p.layers[1].mlp is None and p.layers[2].mixer.chunk is None
    assert FokedraConfig.from_dict(c["Q"]).streams is None and FokedraConfig.from_dict(c["R"]).layers[1].mixer.rot is None
    assert FokedraConfig.from_dict(p.to_dict()) == p
    for spoil, text in ((lambda d: d["layers"][1]["mixer"].update(kv_from=2), "earlier layer"),
                        (lambda d: d["layers"][1]["mixer"].update(dim=32), "differs"),
                        (lambda d: d["layers"][0].update(type="recurrent"), "not a mixer"),
                        (lambda d: d["layers"][0]["mlp"].update(kind="routed"), "kind"),
                        (lambda d: d.update(streams=9), "streams"), (lambda d: d.pop("vocab"), "vocab")):
        bad = json.loads(json.dumps(c["P"]))
        spoil(bad)
        with pytest.raises(ConfigError, match=text):
            FokedraConfig.from_dict(bad)


def test_model_structure_follows_the_configuration():
    from slipstream_b200.config.fokedra_config import FokedraConfig
    from slipstream_b200.models.fokedra import build_fokedra
    model = build_fokedra(FokedraConfig.from_dict(configs()["P"]))
    names = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert names["l0.mix.v"] == (80, 64) and names["l0.mix.o"] == (64, 160) and names["l2.hc2.mix"] == (3, 3)
    assert "l1.mix.k" not in names and "l1.norm2" not in names and "l1.hc2.in" not in names
    # layer 1 reads layer 0's pages under another mask: the group keeps every page; layer 2 has pages of its own
    assert [e.cache_of for e in model.order] == [None, 0, None]
    specs = [(g.spec.head_dim, g.spec.chunk, g.num_entries) for g in model.group_layouts]
    assert specs == [(48, None, 1), (32, None, 1)]
    same = build_fokedra(FokedraConfig.from_dict(configs()["Q"]))
    assert [(g.spec.head_dim, g.spec.chunk, g.num_entries) for g in same.group_layouts] == [(64, None, 1)]
    plainer = json.loads(json.dumps(configs()["Q"]))
    del plainer["layers"][2]
    assert [g.spec.chunk for g in build_fokedra(FokedraConfig.from_dict(plainer)).group_layouts] == [40]


def test_stretched_frequencies_equal_the_plain_table():
    from slipstream_b200.parts import RotaryEncoding, YarnRotaryEncoding
    for dims, base, scaling in ((16, 5000.0, (4.0, 64, 8.0, 0.5)), (64, 300000.0, (3.0, 128, 16.0, 1.0)),
                                (48, 10000.0, (8.0, 4096, 32.0, 1.0)), (8, 50.0, (3.0, 16, 1.0, 0.9))):
        f, m = plain.rotary_frequencies(rot(dims, base, scaling))
        enc = YarnRotaryEncoding(dims + 16, base, dims, interleaved=True, factor=scaling[0], original=scaling[1],
                                 fast=scaling[2], slow=scaling[3])
        assert torch.equal(enc.inverse_frequencies(), f.float()) and enc.mscale == m and not enc.plain
    f, m = plain.rotary_frequencies(rot(32, 100.0))
    assert torch.equal(RotaryEncoding(32, 100.0, 32, interleaved=True, exact_table=True).inverse_frequencies(), f.float())
    assert m == 1.0


def test_chunked_groups_give_pages_back_at_chunk_edges():
    from slipstream_b200.cache import CacheManager, GroupLayout
    from slipstream_b200.parts.base import CacheSpec
    m = CacheManager([GroupLayout(CacheSpec(1, 16, chunk=10), 1)], 6, 4, 2, 1000)
    m.admit("a")
    held = []
    for _ in range(50):
        m.reserve("a", 1)
        m.commit("a", 1)
        held.append(6 - m.num_free_pages())
        length = m.length("a")
        first = (length // 10) * 10 // 4  # the first block the chunk of the next token can still see
        assert m.get("a").first_block[0] == min(first, len(m.get("a").tables[0]))
    assert max(held) <= 4
    m.release("a")
    assert m.all_pages_free()


# --------------------------------------------------------------------------- mechanisms alone

@pytest.mark.gpu
@pytest.mark.parametrize("s, hidden", [(1, 40), (2, 176), (3, 64), (4, 1030), (6, 96)])
def test_hyper_connection_step(s, hidden):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(s * 100 + hidden)
    n = 5
    streams = torch.randn(n, s, hidden, generator=g)
    y = torch.randn(n, hidden, generator=g)
    mix, w_out, w_in = torch.randn(s, s, generator=g), torch.randn(s, generator=g), torch.randn(s, generator=g)
    weight = torch.randn(hidden, generator=g)
    want_streams = plain.hyper_write(streams.double().transpose(0, 1), y.double(), mix.double(), w_out.double())
    want = plain.rms_norm(plain.hyper_read(want_streams, w_in.double()), weight.double(), 1e-5)
    dev = streams.to(DEV)
    got = ops.hc_norm(dev, y.to(DEV), mix.to(DEV), w_out.to(DEV), w_in.to(DEV), weight.to(DEV), 1e-5, torch.float32)
    assert torch.allclose(got.cpu().double(), want, atol=2e-5, rtol=1e-5)
    assert torch.allclose(dev.cpu().double().transpose(0, 1), want_streams, atol=1e-5, rtol=1e-5)
    # a selection of rows leaves the streams alone; no write, plain sum: the model's last norm
    dev = streams.to(DEV)
    rows = torch.tensor([3, 0], dtype=torch.int32, device=DEV)
    got = ops.hc_norm(dev, y.to(DEV), mix.to(DEV), w_out.to(DEV), None, weight.to(DEV), 1e-5, torch.float32, rows=rows)
    want = plain.rms_norm(want_streams.sum(0), weight.double(), 1e-5)[[3, 0]]
    assert torch.allclose(got.cpu().double(), want, atol=2e-5, rtol=1e-5) and torch.equal(dev.cpu(), streams)
    got = ops.hc_norm(dev, None, None, None, w_in.to(DEV), weight.to(DEV), 1e-5, torch.bfloat16 if hidden % 2 == 0 else torch.float32)
    want = plain.rms_norm(plain.hyper_read(streams.double().transpose(0, 1), w_in.double()), weight.double(), 1e-5)
    assert torch.allclose(got.cpu().double(), want, atol=3e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("n_q, n_kv, d, rot_dims, norm_dim, interleaved", [
    (4, 2, 48, 16, 24, True), (3, 1, 64, 64, 64, True), (2, 2, 16, 8, 0, True), (5, 0, 32, 16, 20, True),
    (2, 1, 128, 64, 128, False), (1, 1, 256, 256, 256, True)])
def test_rotation_unit_norm_and_page_write(n_q, n_kv, d, rot_dims, norm_dim, interleaved):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(d + n_q)
    n, page, pages, extra = 9, 4, 7, 24
    real = norm_dim or d  # elements of a head that are not padding
    heads = torch.randn(n, n_q + 2 * n_kv, d, generator=g)
    heads[:, : n_q + n_kv, real:] = 0.0
    rows = torch.cat([heads.reshape(n, -1), torch.randn(n, extra, generator=g)], dim=1)
    positions = torch.tensor([0, 1, 2, 50, 51, 999, 3, 4, 120000], dtype=torch.int32)
    slots = torch.tensor([4, 5, 6, 20, 21, 0, 13, -1, 27], dtype=torch.int32)
    rcfg = rot(rot_dims, 777.0, (3.0, 32, 4.0, 0.5))
    f, mscale = plain.rotary_frequencies(rcfg)
    kv = torch.zeros(pages, 2, max(n_kv, 1), page, d)
    dev_rows, dev_kv = rows.to(DEV), kv.to(DEV)
    ops.rope_norm_cache(dev_rows, positions.to(DEV), slots.to(DEV), f.float().to(DEV), dev_kv if n_kv else None, n_q, n_kv, d,
                        rot_dims, interleaved=interleaved, mscale=mscale, norm_dim=norm_dim, eps=1e-6)
    qk = heads[:, : n_q + n_kv, :real].double()
    if interleaved:
        turned = plain.rotate_pairs(qk, positions, rcfg)
    else:  # half-split pairs, restated here: element i with element i + rot_dims / 2
        angle = positions.double()[:, None] * f[None, :]
        c, s_ = (torch.cos(angle) * mscale)[:, None, :], (torch.sin(angle) * mscale)[:, None, :]
        a, b = qk[..., : rot_dims // 2], qk[..., rot_dims // 2: rot_dims]
        turned = torch.cat([a * c - b * s_, b * c + a * s_, qk[..., rot_dims:]], dim=-1)
    if norm_dim:
        turned = plain.rms_unit(turned, 1e-6)
    out = dev_rows.cpu()
    got = out[:, : (n_q + 2 * n_kv) * d].view(n, -1, d)
    # a float32 angle is off by up to 6e-8 of itself: 7e-3 rad at position 120,000
    tol = [2e-5 + 5e-7 * int(p) for p in positions]
    for t in range(n):
        assert torch.allclose(got[t, :n_q, :real].double(), turned[t, :n_q], atol=tol[t]), t
        assert torch.equal(got[t, :n_q, real:], torch.zeros(n_q, d - real))
    assert torch.equal(out[:, (n_q + 2 * n_kv) * d:], rows[:, (n_q + 2 * n_kv) * d:])  # what follows the heads is left alone
    cache = dev_kv.cpu()
    for t in range(n):
        if n_kv == 0:
            continue
        if slots[t] < 0:  # no slot: the key is rotated in place
            assert torch.allclose(got[t, n_q: n_q + n_kv, :real].double(), turned[t, n_q:], atol=tol[t])
            continue
        pg, off = int(slots[t]) // page, int(slots[t]) % page
        assert torch.allclose(cache[pg, 0, :, off, :real].double(), turned[t, n_q:], atol=tol[t])
        assert torch.equal(cache[pg, 1, :, off], heads[t, n_q + n_kv:])
    used = {(int(s) // page, int(s) % page) for s in slots if s >= 0}
    for pg in range(pages):
        for off in range(page):
            if (pg, off) not in used:
                assert not cache[pg, :, :, off].any()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_limited_gated_unit_and_sigmoid_gate(dtype):
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(3)
    for inter, block, limit in ((80, 80, 1.0), (128, 64, 2.5), (24, 8, 0.3)):
        gate, up = (torch.randn(6, inter, generator=g) * 2).to(dtype), (torch.randn(6, inter, generator=g) * 2).to(dtype)
        stacked = torch.stack([gate.view(6, -1, block), up.view(6, -1, block)], dim=2).reshape(6, 2 * inter)
        got = ops.glu_limited(stacked.to(DEV).contiguous(), block, 1.702, limit, 1.0).cpu().double()
        gl, ul = gate.double().clamp(max=limit), up.double().clamp(-limit, limit)
        want = gl * torch.sigmoid(1.702 * gl) * (ul + 1.0)
        assert torch.allclose(got, want, atol=1e-6 if dtype == torch.float32 else 2e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)
    x, gates = torch.randn(5, 48, generator=g).to(dtype), torch.randn(5, 100, generator=g).to(dtype)
    dev = x.to(DEV)
    ops.sigmoid_gate(dev, gates.to(DEV)[:, 52:])
    want = x.double() * torch.sigmoid(gates.double()[:, 52:])
    assert torch.allclose(dev.cpu().double(), want, atol=1e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("tokens, inter, k", [(5, 256, 200), (16, 1024, 64), (2048, 9472, 128), (40, 128, 72)])
def test_gated_unit_in_the_products_epilogue(tokens, inter, k):
    """Few tokens (the streaming product), many tokens and features (the two-SM product) and a case that takes
    the product followed by the activation kernel: all against the plain formula on the bfloat16 inputs."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(tokens)
    x = (torch.randn(tokens, k, generator=g)).bfloat16()
    gate = (torch.randn(inter, k, generator=g) * 2.0 * k ** -0.5).bfloat16()
    up = (torch.randn(inter, k, generator=g) * 2.0 * k ** -0.5).bfloat16()
    stacked = torch.stack([gate.view(-1, 64, k), up.view(-1, 64, k)], dim=1).reshape(2 * inter, k).contiguous()
    got = ops.gate_up_glu(x.to(DEV), stacked.to(DEV), None, 64, 1.702, 1.5, 1.0).cpu().double()
    want = plain.dense_ff(x.double(), {"gate": gate.double(), "up": up.double(), "down": torch.eye(inter, dtype=torch.float64)},
                          {"limit": 1.5})
    assert got.shape == want.shape and torch.allclose(got, want, atol=3e-2, rtol=2e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("s, tokens, hidden, k", [(1, 3, 128, 512), (2, 8, 256, 128), (3, 16, 384, 1024), (4, 1, 128, 256),
                                                 (3, 5, 320, 256), (5, 4, 128, 256), (2, 40, 128, 256)])
def test_a_products_write_into_the_streams(s, tokens, hidden, k):
    """A branch's last projection with the write into the streams and the next read + norm: inside the product where
    it can (few bfloat16 tokens, at most 4 streams, a width in steps of 128), else product then kernel; either way
    the streams, the norm (as a tensor, or pending and then finished by hand or by the next product) are the plain ones."""
    from slipstream_b200 import ops
    g = torch.Generator().manual_seed(s * 1000 + hidden)
    x = torch.randn(tokens, k, generator=g).bfloat16()
    w = (torch.randn(hidden, k, generator=g) * k ** -0.5).bfloat16()
    streams = torch.randn(tokens, s, hidden, generator=g)
    mix, w_out, w_in = torch.randn(s, s, generator=g), torch.randn(s, generator=g), torch.randn(s, generator=g)
    weight = (1.0 + 0.1 * torch.randn(hidden, generator=g)).bfloat16()
    host = torch.cat([mix.reshape(-1), w_out, w_in]).numpy().copy()
    y = (x.double() @ w.double().T).bfloat16().double()  # the branch output is rounded to bfloat16 before it is written
    want_streams = plain.hyper_write(streams.double().transpose(0, 1), y, mix.double(), w_out.double())
    want = plain.rms_norm(plain.hyper_read(want_streams, w_in.double()), weight.double(), 1e-6)
    dev = streams.to(DEV)
    got = ops.linear_hc_rmsnorm(x.to(DEV), w.to(DEV), None, dev, mix.to(DEV), w_out.to(DEV), w_in.to(DEV), host,
                                weight.to(DEV), 1e-6, torch.bfloat16)
    fused = isinstance(got, ops.PendingNorm)
    assert fused == (s <= 4 and tokens <= 16 and hidden % 128 == 0)
    assert torch.allclose(dev.cpu().double().transpose(0, 1), want_streams, atol=2e-2, rtol=1e-2)
    if fused:
        # the next product finishes the norm: against the plain norm times a matrix
        w2 = (torch.randn(256, hidden, generator=g) * hidden ** -0.5).bfloat16()
        out = ops.linear(got, w2.to(DEV)).cpu().double()
        assert torch.allclose(out, want @ w2.double().T, atol=4e-2, rtol=2e-2)
        got = got.materialize()
    assert torch.allclose(got.cpu().double(), want, atol=4e-2, rtol=2e-2)


def chunked_attention_plain(q, k, v, chunk, scale):
    """q [n, H, d] at the LAST n of the m positions of k, v [m, G, d]."""
    n, H, _ = q.shape
    m, G, _ = k.shape
    see = plain.visible(m, {"size": chunk} if chunk else None)[m - n:]
    out = torch.empty(n, H, v.shape[-1], dtype=torch.float64)
    for h in range(H):
        score = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        out[:, h] = torch.softmax(score.masked_fill(~see, float("-inf")), dim=-1) @ v[:, h // (H // G)].double()
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("d, page, chunk, lens, q_lens", [
    (48, 16, 110, (111, 220, 109, 331), (1, 1, 1, 1)),      # decode: just behind, at and in front of an edge
    (64, 16, 40, (81, 80, 79, 200), (1, 1, 1, 1)),          # the TMA-fed decode kernel with a lower bound
    (64, 8, 40, (90, 130, 41), (50, 130, 2)),               # prompt portions across edges
    (128, 16, 100, (700, 333, 64), (300, 333, 1)), (64, 32, 64, (640,), (640,)), (64, 16, 1000, (300, 90), (300, 2)),
    (32, 4, 7, (30, 64, 15), (9, 64, 15)), (16, 16, 1, (20, 5), (20, 1)), (48, 16, 110, (500,), (260,))])
def test_chunked_visibility_in_every_attention_kernel(d, page, chunk, lens, q_lens):
    from slipstream_b200 import ops
    from slipstream_b200.engine.context import query_tiles_host
    g = torch.Generator().manual_seed(d + chunk)
    n_q, n_kv, scale = 4, 2, 0.9
    blocks = [-(-m // page) for m in lens]
    order = torch.randperm(sum(blocks) + 3, generator=g).tolist()
    table = torch.full((len(lens), max(blocks)), -1, dtype=torch.int32)
    kv = torch.randn(sum(blocks) + 3, 2, n_kv, page, d, generator=g)  # unused slots hold noise, not zeros
    ks, vs, want, qs = [], [], [], []
    for r, (m, n) in enumerate(zip(lens, q_lens)):
        k, v, q = torch.randn(m, n_kv, d, generator=g), torch.randn(m, n_kv, d, generator=g), torch.randn(n, n_q, d, generator=g)
        for b in range(blocks[r]):
            table[r, b] = order.pop()
            part = slice(b * page, min(m, (b + 1) * page))
            kv[table[r, b], 0, :, : part.stop - part.start] = k[part].transpose(0, 1)
            kv[table[r, b], 1, :, : part.stop - part.start] = v[part].transpose(0, 1)
        want.append(chunked_attention_plain(q.bfloat16(), k.bfloat16(), v.bfloat16(), chunk, scale).reshape(n, n_q * d))
        qs.append(q.reshape(n, n_q * d))
    want, q = torch.cat(want), torch.cat(qs)
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    seq = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tables = table.to(DEV)
    import numpy as np
    for dtype in (torch.float32, torch.bfloat16):
        qd, kvd = q.bfloat16().to(dtype).to(DEV), kv.bfloat16().to(dtype).to(DEV)
        out = torch.zeros_like(qd)
        if dtype == torch.float32:
            req, q0 = query_tiles_host(np.asarray(q_lens), 16)
            ops.paged_attention_simt(qd, n_q * d, out, kvd, tables, torch.from_numpy(req).to(DEV), torch.from_numpy(q0).to(DEV),
                                     q_start, seq, n_q, n_kv, d, scale, chunk=chunk)
            assert torch.allclose(out.cpu().double(), want, atol=2e-5)
            continue
        req, row0 = query_tiles_host(np.asarray(q_lens) * (n_q // n_kv), 64)
        ops.paged_attention_prefill(qd, n_q * d, out, kvd, tables, torch.from_numpy(req).to(DEV), torch.from_numpy(row0).to(DEV),
                                    q_start, seq, n_q, n_kv, d, scale, chunk=chunk)
        assert torch.allclose(out.cpu().double(), want, atol=3e-2)
        if d in (64, 128):  # the tcgen05 kernel: tiles of 128 / group tokens, alone and with the keys in two parts
            from slipstream_b200.engine.context import query_tiles_longest_first_host
            treq, tok0 = query_tiles_longest_first_host(np.asarray(q_lens), np.asarray(lens), 128 // (n_q // n_kv))
            for parts in (1, 2):
                out = torch.zeros_like(qd)
                ops.paged_attention_prefill_tcgen05(qd, n_q * d, out, kvd, tables, torch.from_numpy(treq).to(DEV),
                                                    torch.from_numpy(tok0).to(DEV), q_start, seq, n_q, n_kv, d, scale, parts,
                                                    chunk=chunk)
                assert torch.allclose(out.cpu().double(), want, atol=3e-2), parts
        if max(q_lens) == 1:
            for slices in (1, 2, 4):
                for tma in ((False, True) if d in (64, 128) else (False,)):
                    out = torch.zeros_like(qd)
                    ops.paged_attention_decode(qd, n_q * d, out, kvd, tables, q_start, seq, len(lens), n_q, n_kv, d, scale,
                                               n_slices=slices, tma=tma, chunk=chunk)
                    assert torch.allclose(out.cpu().double(), want, atol=3e-2), (slices, tma)
    ops.check_errors(DEV)


# --------------------------------------------------------------------------- whole models

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q", "R", "T", "U"])
def test_every_way_of_cutting_gives_the_plain_logits(models, name, dtype):
    """Whole prompts, token-by-token decoding from the first token on, portions down to two tokens, and unequal
    requests side by side while others come and go, in a pool that holds less than the requests need in total."""
    folder, config, weights = models[name]
    reqs = {"a": tokens_of(config["vocab"], 97, 1), "b": tokens_of(config["vocab"], 45, 2),
            "c": tokens_of(config["vocab"], 1, 3), "d": tokens_of(config["vocab"], 130, 4), "e": tokens_of(config["vocab"], 33, 5)}
    want = {k: plain_logits(name, config, weights, v) for k, v in reqs.items()}
    runner = make_runner(folder, dtype, pages=18, page=16)  # 288 token slots for 306 tokens: pages come back and go out again
    plans = {
        "whole": [[(k, len(v))] for k, v in reqs.items()],
        "token by token": [[("b", 1)] for _ in range(45)] + [[("c", 1)]],
        "portions": [[("a", n)] for n in (2, 30, 2, 5, 16, 2, 40)] + [[("d", n)] for n in (64, 2, 62, 2)],
        "mixed": [[("a", 50), ("c", 1), ("b", 3)], [("a", 2), ("b", 2)], [("b", 38), ("a", 1)], [("a", 1), ("b", 1), ("e", 20)],
                  [("a", 43), ("b", 1), ("e", 2)], [("e", 1), ("d", 70)], [("d", 2), ("e", 10)], [("d", 58)]],
    }
    for what, plan in plans.items():
        got = replay(runner, reqs, plan)
        for k, v in got.items():
            dist = distance(v, want[k][: v.shape[0]])
            assert dist < BOUND[dtype], (what, k)
        assert runner.cache.all_pages_free() and runner.cache.num_free_slots() == 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_crosses_chunks_and_pages(models, dtype):
    """A short prompt and 150 decoded tokens (captured decode steps), beside a second request that joins and leaves:
    every chunk edge of 7, 16, 32 and 40 and every page edge of 8 is crossed in decoding."""
    for name in ("P", "Q", "R", "T"):
        folder, config, weights = models[name]
        reqs = {"a": tokens_of(config["vocab"], 160, 7), "b": tokens_of(config["vocab"], 60, 8)}
        want = {k: plain_logits(name, config, weights, v) for k, v in reqs.items()}
        runner = make_runner(folder, dtype, pages=30, page=8)
        plan = [[("a", 10)]] + [[("a", 1)] for _ in range(40)] + [[("a", 1), ("b", 12)]] + [[("a", 1), ("b", 1)] for _ in range(48)]
        plan += [[("a", 1)] for _ in range(150 - 89)]
        got = replay(runner, reqs, plan)
        for k in reqs:
            dist = distance(got[k], want[k])
            assert dist < BOUND[dtype], (name, k)


@pytest.mark.gpu
def test_a_key_that_should_not_be_seen_would_show(models):
    """The bounds above are meaningful: the plain logits with a chunk size off by one differ from the right ones by
    far more than the bounds allow."""
    folder, config, weights = models["Q"]
    toks = tokens_of(config["vocab"], 97, 1)
    right = plain.forward(config, weights, toks)[0]
    wrong = json.loads(json.dumps(config))
    wrong["layers"][0]["mixer"]["mask"]["size"] = 41
    assert distance(plain.forward(wrong, weights, toks)[0].float(), right) > 5 * BOUND["bfloat16"]


@pytest.mark.gpu
def test_greedy_generation_through_the_engine(models):
    """The package's entry point and scheduler: several requests at once, prompts in portions of 16, pages that come
    back; every generated token is the plain implementation's arg-max (or within a hair of it)."""
    from slipstream_b200 import CacheConfig, EngineConfig, SamplingParams, SchedulerConfig
    from slipstream_b200.engine.llm_engine import LLMEngine, Request
    for name, dtype, slack in (("P", "float32", 1e-4), ("Q", "bfloat16", 3e-2)):
        folder, config, weights = models[name]
        engine = LLMEngine(EngineConfig.for_model(folder, dtype=dtype, max_model_len=512,
                                                  cache=CacheConfig(block_size=8, num_gpu_blocks=40),
                                                  scheduler=SchedulerConfig(prefill_chunk_size=16, max_num_seqs=4)))
        prompts = [tokens_of(config["vocab"], n, 20 + n) for n in (1, 9, 37, 50, 23)]
        params = SamplingParams(max_tokens=14, temperature=0.0, ignore_eos=True)
        outs = engine.generate_batch([Request(f"r{i}", None, p, params, float(i)) for i, p in enumerate(prompts)])
        for prompt, out in zip(prompts, outs):
            assert len(out) == 14
            toks = list(prompt)
            for tok in out:
                logits = plain.forward(config, weights, toks)[0][-1]
                assert logits[tok] >= logits.max() - slack * logits.abs().max(), (name, len(toks))
                toks.append(tok)
        assert engine.runner.cache.all_pages_free()
        engine.runner.check()
