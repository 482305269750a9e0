"""Murutar through the engine against the plain implementation.

Replays through bin/trace_run: the same requests whole, with their last tokens one by one, in
portions of changing size down to two tokens, and mixed (up to four live, portions beside single
tokens, few pages and four state slots so that both are used again, freed pages filled with NaN),
in float32 and bfloat16, also from captured CUDA graphs.  "Sharp" variants scale queries and keys
so that a lost far token, a key on the wrong side of a window's edge or a lost state shows.
Generation through LLMEngine and ContinuousBatchingEngine.  The kernels one by one."""
import math
from types import SimpleNamespace

import pytest
import torch

import murutar_util as mu
import plain_murutar as plain
import replay_util as ru

pytestmark = pytest.mark.gpu

LENGTHS = {"mix": [1, 9, 40, 131, 260], "odd": [2, 17, 64, 150], "wide": [3, 33, 97, 230],
           "only_attention": [1, 23, 24, 25, 70], "only_lightning": [1, 2, 45, 100]}
LENGTHS.update({k + "_dense": v for k, v in LENGTHS.items()})


CLOSE_CALL = 0.08  # difference of router logits below which bfloat16 activations may route a token otherwise


def first_close_call(config, weights, ids):
    """(logits, first position at which the plain router's choice hangs on less than CLOSE_CALL)."""
    plain.ROUTING_MARGINS = []
    try:
        logits = plain.forward(config, weights, ids)[0].float()
        close = [t for t, m in plain.ROUTING_MARGINS if m < CLOSE_CALL]
    finally:
        plain.ROUTING_MARGINS = None
    return logits, (min(close) if close else len(ids))


def replay(name, dtype, tmp_path, cuda_graph=False, sharp=False):
    """float32: every position within 2e-4.  bfloat16: within rounding; from the first position of
    a request at which the plain router's choice is a close call, the engine may have sent a token
    to another expert, which later tokens see through the caches and states: those positions are
    held to six times the bound (a lost key, state or page is far beyond that)."""
    spec = mu.CONFIGS[name]
    model_dir = str(tmp_path / "model")
    config, weights = mu.make_folder(model_dir, name, sharp=sharp)
    prompts = {f"p{n}": ru.random_ids(n, config["vocab"], 100 + n) for n in LENGTHS[name]}
    trace, peak = ru.build_four_mode_trace(prompts, spec["page_size"])
    got = ru.run_trace(model_dir, dtype, trace, peak, str(tmp_path / "out"), page_size=spec["page_size"],
                       cuda_graph=cuda_graph, max_requests=4)
    refs = {n: first_close_call(config, weights, ids) for n, ids in prompts.items()}
    modes, strict = set(), 0
    for (step, rid, pos), row in got.items():
        mode, pname = rid.split("/")
        modes.add(mode.rstrip("01"))
        ref = refs[pname][0][pos]
        assert torch.isfinite(row).all(), (step, rid, pos)
        err = (row - ref).abs().max().item()
        scale = max(ref.abs().max().item(), 1e-3)
        if dtype == "float32":
            assert err <= 2e-4 * max(scale, 1.0), f"first wrong place: step {step} request {rid} position {pos}: {err}"
        else:
            loose = 1.0 if pos < refs[pname][1] else 6.0
            strict += loose == 1.0
            assert err <= loose * (0.04 * scale + 0.03), f"first wrong place: step {step} request {rid} position {pos}: {err}"
    assert modes == {"whole", "tail", "portions", "mixed"}
    return strict / max(len(got), 1)


def without_experts(name):
    """The configuration with every mixture of experts replaced by a dense feed-forward: no routing,
    so bfloat16 is held to the strict bound everywhere."""
    import copy
    spec = copy.deepcopy(mu.CONFIGS[name])
    for e in spec["config"]["layers"]:
        if e.get("mlp") and e["mlp"]["kind"] == "moe":
            e["mlp"] = mu.dense(2 * e["mlp"]["expert"]["ff"], limit=1.2)
    mu.CONFIGS[name + "_dense"] = spec
    return name + "_dense"


@pytest.mark.parametrize("name", sorted(mu.CONFIGS))
def test_replay_float32(name, tmp_path):
    replay(name, "float32", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_replay_bfloat16(name, tmp_path):
    replay(name, "bfloat16", tmp_path)


@pytest.mark.parametrize("name", ["mix", "odd", "wide"])
def test_replay_bfloat16_without_experts_is_within_rounding_everywhere(name, tmp_path):
    assert replay(without_experts(name), "bfloat16", tmp_path) == 1.0


@pytest.mark.parametrize("name", ["mix", "wide"])
def test_replay_bfloat16_single_token_steps_from_captured_graphs(name, tmp_path):
    replay(name, "bfloat16", tmp_path, cuda_graph=True)


@pytest.mark.parametrize("name", ["mix", "odd", "only_attention", "only_lightning"])
def test_replay_float32_sharp_window_edges_and_long_memories(name, tmp_path):
    replay(name, "float32", tmp_path, sharp=True)


# ------------------------------------------------------------------ generation entry points
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("mix", "wide"):
        d = str(tmp_path_factory.mktemp(f"murutar_{name}"))
        out[name] = (d,) + mu.make_folder(d, name)
    return out


def load(folder, dtype):
    from dispec_b200 import load_model
    return load_model(folder, dtype, "cuda:0")


def assert_greedy(weights, config, prompt, got, dtype):
    """Teacher-forced on the engine's tokens: each equals the plain argmax, or the plain top-2 gap
    there is below what the type can resolve."""
    logits = plain.forward(config, weights, list(prompt) + list(got))[0].float()
    for i, tok in enumerate(got):
        row = logits[len(prompt) - 1 + i]
        top2 = torch.topk(row, 2)
        reach = 1e-4 if dtype == "float32" else 2 * (0.03 * row.abs().max().item() + 0.02)
        assert tok == int(top2.indices[0]) or float(top2.values[0] - top2.values[1]) < reach, (i, tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_llm_engine(folders, dtype):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix"]
    engine = LLMEngine(load(folder, dtype), num_blocks=32, cuda_graph=dtype == "bfloat16")
    for n in (1, 9, 40):  # the same engine: pages and the state slot are used again
        prompt = ru.random_ids(n, config["vocab"], 300 + n)
        got = engine.generate(prompt, 10, SamplingParams(temperature=0.0))
        assert len(got) == 10
        assert_greedy(weights, config, prompt, got, dtype)
    cache = engine.runner.cache
    assert all(cache.num_free_pages(g) == 32 for g in range(len(cache.groups))) and cache.free_slots() == 4


def test_long_decoding_float32_past_every_window(folders):
    from dispec_b200 import LLMEngine, SamplingParams
    folder, config, weights = folders["mix"]
    engine = LLMEngine(load(folder, "float32"), num_blocks=32)
    prompt = ru.random_ids(3, config["vocab"], 1)
    got = engine.generate(prompt, 200, SamplingParams())
    assert len(got) == 200
    assert_greedy(weights, config, prompt, got, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_continuous_batching_more_requests_than_slots(folders, dtype):
    """Seven requests through three state slots and a small pool: portions of prompts beside
    decoded tokens; slots and pages of finished requests go to waiting ones."""
    from dispec_b200 import ContinuousBatchingEngine, KVConfig, SamplingParams
    folder, config, weights = folders["wide"]
    engine = ContinuousBatchingEngine(load(folder, dtype), KVConfig(block_size=32), num_blocks=12,
                                      max_batch_tokens=48, chunk_size=20, max_num_seqs=3)
    reqs = []
    for i, n in enumerate([1, 9, 40, 64, 9, 70, 2]):
        prompt = ru.random_ids(n, config["vocab"], 400 + i)
        reqs.append((engine.add_request(prompt, 9, SamplingParams(temperature=0.0)), prompt))
    engine.run_until_done()
    out = engine.collect_outputs()
    for rid, prompt in reqs:
        assert len(out[rid]) == 9
        assert_greedy(weights, config, prompt, out[rid], dtype)
    assert engine.runner.cache.free_slots() == 3


# ----------------------------------------------------------------------- kernels one by one
def dev(t, dtype=torch.float32):
    return t.to(device="cuda:0", dtype=dtype).contiguous()


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda:0")


@pytest.mark.parametrize("width", [52, 256, 1000])
def test_layer_norm_and_stream_update_kernels(width):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3 + 1.5
    y, gate = torch.randn(7, width, generator=g), torch.randn(7, width, generator=g) * 2
    w, ls, rw = (1 + 0.1 * torch.randn(width, generator=g) for _ in range(3))
    got = norm32.layer_norm(dev(x), dev(w), 1e-5, torch.float32)
    assert (got.cpu().double() - plain.layer_norm(x.double(), w.double(), 1e-5)).abs().max() < 1e-5
    rows = i32([5, 0, 5])
    got = norm32.layer_norm(dev(x), dev(w), 1e-5, torch.bfloat16, rows=rows)
    assert (got.float().cpu().double() - plain.layer_norm(x.double(), w.double(), 1e-5)[[5, 0, 5]]).abs().max() < 0.03
    # gated and scaled addend, then the next norm
    xs = dev(x)
    h = norm32.stream_update(xs, dev(y), gate=dev(gate), scale=dev(ls), norm_weight=dev(w), norm_eps=1e-5,
                             out_dtype=torch.float32)
    want = x.double() + y.double() * ls.double() * torch.sigmoid(gate.double())
    assert (xs.cpu().double() - want).abs().max() < 1e-5
    assert (h.cpu().double() - plain.layer_norm(want, w.double(), 1e-5)).abs().max() < 1e-5
    # RMS-normed addend, then a rounded copy; then a plain addend and nothing else
    r = norm32.stream_update(xs, dev(y), rms_weight=dev(rw), rms_eps=1e-6, out_dtype=torch.bfloat16)
    want = want + plain.rms_norm(y.double(), rw.double(), 1e-6)
    assert (xs.cpu().double() - want).abs().max() < 1e-5
    assert (r.float().cpu().double() - want).abs().max() < 0.05 and r.dtype == torch.bfloat16
    assert norm32.stream_update(xs, dev(y, torch.bfloat16)) is None
    assert (xs.cpu().double() - (want + y.bfloat16().double())).abs().max() < 1e-5


def test_activation_table_gate_softcap_and_embedding_kernels():
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(6)
    z = torch.randn(5, 2 * 33, generator=g) * 2
    got = norm32.clamped_glu(dev(z), 0.8, 1.702, torch.float32)
    gg, uu = z[:, :33].double().clamp(max=0.8), z[:, 33:].double().clamp(-0.8, 0.8)
    assert (got.cpu().double() - gg * torch.sigmoid(1.702 * gg) * (uu + 1)).abs().max() < 1e-6
    table = torch.randn(11, 12, generator=g)
    ids = [3, 0, 10, 3, 7]
    zz = torch.randn(5, 4, generator=g) * 2
    got = norm32.gelu_table_gate(dev(zz), dev(table, torch.bfloat16), 8, i32(ids), torch.float32)
    want = plain.gelu_tanh(zz.double()) * table.bfloat16().double()[ids][:, 8:12]
    assert (got.cpu().double() - want).abs().max() < 1e-6
    x = torch.randn(3, 50, generator=g) * 40
    got = norm32.softcap_(dev(x), 30.0)
    assert (got.cpu().double() - 30 * torch.tanh(x.double() / 30)).abs().max() < 1e-4
    emb = norm32.embed_scaled(dev(table, torch.bfloat16), i32(ids), 3.5)
    assert emb.dtype == torch.float32 and torch.equal(emb.cpu(), table.bfloat16().float()[ids] * 3.5)


@pytest.mark.parametrize("E,groups,keep,top", [(6, 3, 2, 2), (9, 3, 3, 4), (16, 4, 2, 3), (4, 1, 1, 1), (40, 5, 1, 8),
                                               (8, 8, 3, 3)])
def test_router_kernel_chooses_what_the_plain_router_chooses(E, groups, keep, top):
    from dispec_b200.ops import moe
    g = torch.Generator().manual_seed(E)
    T, W = 37, 29
    h = torch.randn(T, W, generator=g)
    w = torch.randn(E, W, generator=g)
    ids, wts = moe.route(dev(h), dev(w), groups, keep, top)
    router = {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}
    for t in range(T):
        s = torch.softmax(w.double() @ h[t].double(), dim=0)
        want = plain.route(s, router).tolist()
        got = ids[t].tolist()
        assert sorted(got) == sorted(want), t
        assert (wts[t].cpu().double() - s[got]).abs().max() < 1e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,ff,E,groups,keep,top", [(1, 20, 6, 4, 1, 1, 1), (45, 52, 14, 9, 3, 3, 4),
                                                     (150, 64, 40, 6, 3, 2, 2), (70, 128, 96, 16, 4, 2, 3)])
def test_mixture_of_experts_feed_forward(dtype, T, W, ff, E, groups, keep, top):
    """The part itself: router, rows sorted by expert on the device, both products, the weighted
    sum.  More than one tile of rows per expert, experts that nobody chooses."""
    from dispec_b200.parts.moe import GroupedMoE
    g = torch.Generator().manual_seed(T)
    part = GroupedMoE(W, ff, E, top, groups, keep)
    w = {"router": (3 * torch.randn(E, W, generator=g) / W ** 0.5)}
    for e in range(E):
        w[f"e{e}.up"] = (torch.randn(ff, W, generator=g) / W ** 0.5).bfloat16().float()
        w[f"e{e}.down"] = (torch.randn(W, ff, generator=g) / ff ** 0.5).bfloat16().float()
    tensors = {"router.weight": dev(w["router"])}
    for e in range(E):
        tensors[f"experts.{e}.up.weight"] = dev(w[f"e{e}.up"], dtype)
        tensors[f"experts.{e}.down.weight"] = dev(w[f"e{e}.down"], dtype)
    part.load(tensors)
    h = torch.randn(T, W, generator=g).bfloat16().float()
    got = part.forward(SimpleNamespace(dtype=dtype), dev(h, dtype)).cpu().double()
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}}
    want = plain.moe_ff(h.double(), {"x." + k: v.double() for k, v in w.items()}, "x.", mlp)
    tol = 1e-4 if dtype == torch.float32 else 0.03
    assert (got - want).abs().max() < tol * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("H,d,dv", [(1, 10, 7), (2, 64, 48), (2, 160, 40), (3, 32, 130)])
def test_lightning_recurrence_carries_its_state_over_cuts(H, d, dv):
    """Two requests of unequal length, whole and cut at arbitrary places down to single tokens,
    in state slots that are not neighbours: outputs and final states agree with the plain form."""
    from dispec_b200.ops import recurrence as R
    g = torch.Generator().manual_seed(H * 100 + d)
    lens, slots = [37, 5], [2, 0]
    proj = [torch.randn(n, 2 * H * d + H * dv, generator=g) for n in lens]
    decay = [0.9, 1.0, 0.99][:H]

    def plain_run(p):
        n = p.shape[0]
        q, k, v = (plain.silu(p[:, :H * d].double()).view(n, H, d), plain.silu(p[:, H * d:2 * H * d].double()).view(n, H, d),
                   plain.silu(p[:, 2 * H * d:].double()).view(n, H, dv))
        o, S = plain.lightning_recurrence(q, k, v, decay)
        return o.reshape(n, -1), S

    want = [plain_run(p) for p in proj]
    for cuts in ([[37], [5]], [[2, 16, 1, 18], [3, 2]]):
        state = torch.full((4, H, d, dv), float("nan"), device="cuda:0")
        state[slots] = 0.0
        got, done = [[], []], [0, 0]
        for step in range(max(len(c) for c in cuts)):
            rows, starts, sl, pos, who = [], [0], [], [], []
            for s in (1, 0):
                if step < len(cuts[s]):
                    n = cuts[s][step]
                    rows.append(proj[s][done[s]:done[s] + n])
                    pos += list(range(done[s], done[s] + n))
                    starts.append(starts[-1] + n)
                    sl.append(slots[s])
                    who.append((s, n))
                    done[s] += n
            o = R.linear_recurrence(dev(torch.cat(rows)), 0, H * d, 2 * H * d, R.FIXED_DECAY, H, d, dv, state, i32(sl),
                                    i32(starts), i32(pos), decay=dev(torch.tensor(decay)), silu_inputs=True)
            at = 0
            for s, n in who:
                got[s].append(o[at:at + n].cpu())
                at += n
        for s in (0, 1):
            tol = 1e-4 * max(1.0, want[s][0].abs().max().item())
            assert (torch.cat(got[s]).double() - want[s][0]).abs().max() < tol, (cuts, s)
            assert (state[slots[s]].cpu().double() - want[s][1]).abs().max() < tol
        assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all()


@pytest.mark.parametrize("n", [60, 1536])
def test_whole_row_norm_with_sigmoid_gate(n):
    from dispec_b200.ops import norm32
    g = torch.Generator().manual_seed(8)
    o, gate, gain = torch.randn(5, n, generator=g) * 3, torch.randn(5, n, generator=g), torch.rand(n, generator=g) + 0.5
    y = norm32.head_norm_gate(dev(o), 1, 1e-6, torch.float32, gain=dev(gain), gate=dev(gate), gate_kind="sigmoid")
    want = plain.rms_norm(o.double(), gain.double(), 1e-6) * torch.sigmoid(gate.double())
    assert (y.cpu().double() - want).abs().max() < 1e-5


def _cache(k_pool, v_pool, table, write=True):
    return SimpleNamespace(key_pool=k_pool, value_pool=v_pool, page_table=table, write=write,
                           tensors={"key": k_pool, "value": v_pool})


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
def test_rotate_blend_and_store_kernel(pool_dtype):
    from dispec_b200.ops import attention as A
    g = torch.Generator().manual_seed(2)
    H, G, dk, dv, page, rot = 3, 2, 10, 6, 4, 6
    cols = (H + G) * dk + G * dv
    qkv = torch.randn(6, cols, generator=g)
    other = torch.randn(6, G * dv, generator=g)
    pos = torch.tensor([3, 4, 5, 0, -1, 9], dtype=torch.int32)
    seq = torch.tensor([0, 0, 0, 1, 1, 1], dtype=torch.int32)
    table = torch.tensor([[2, 0, -1], [1, 3, 4]], dtype=torch.int32)
    inv_freq = (20.0 ** (-torch.arange(0, rot, 2).double() / rot)).float()
    lam = torch.tensor(0.3)
    for blend in (False, True):
        k_pool = torch.full((5, G, page, dk), float("nan"), device="cuda:0", dtype=pool_dtype)
        v_pool = torch.full((5, G, page, dv), float("nan"), device="cuda:0", dtype=pool_dtype)
        q = A.qkv_rotate_store(dev(qkv), pos.cuda(), seq.cuda(), _cache(k_pool, v_pool, table.cuda()), dev(inv_freq), rot,
                               H, G, dk, dv, pool_dtype, v_other=dev(other) if blend else None,
                               blend=dev(lam) if blend else None)
        tol = 1e-5 if pool_dtype == torch.float32 else 0.03
        written = 0
        for t in range(6):
            if pos[t] < 0:
                continue
            p1 = pos[t:t + 1]
            want_q = plain.rotate_halves(qkv[t, :H * dk].double().view(1, H, dk), p1, rot, 20.0)[0]
            want_k = plain.rotate_halves(qkv[t, H * dk:(H + G) * dk].double().view(1, G, dk), p1, rot, 20.0)[0]
            want_v = qkv[t, (H + G) * dk:].double().view(G, dv)
            if blend:
                want_v = 0.7 * want_v + 0.3 * other[t].double().view(G, dv)
            pg, off = int(table[seq[t], pos[t] // page]), int(pos[t] % page)
            assert (q[t].float().cpu().double().view(H, dk) - want_q).abs().max() < tol
            assert (k_pool[pg, :, off].float().cpu().double() - want_k).abs().max() < tol
            assert (v_pool[pg, :, off].float().cpu().double() - want_v).abs().max() < tol
            written += 1
        assert int(torch.isfinite(k_pool[:, 0, :, 0].float()).sum()) == written  # nothing else was touched


def _aimed_attention_case(H, G, dk, dv, page, window, seed):
    """Stored keys of one request on scattered pages (NaN elsewhere) and queries that are each
    aimed at one key: the first token, both sides of a page border, the window's first key and
    the one before it (outside), the query's own position and the one after it (stored already,
    as in a portion of a prompt), and one aimed at nothing, where the sink takes the weight."""
    g = torch.Generator().manual_seed(seed)
    n = 7 * page + 3
    n_pages = 11
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.tensor([order[:8]], dtype=torch.int32)
    keys = torch.randn(n, G, dk, generator=g).bfloat16().float()
    vals = torch.randn(n, G, dv, generator=g).bfloat16().float()
    p = n - 2
    lo = max(0, p - window + 1) if window else 0
    cases = [(p, 0), (p, page - 1), (p, page), (p, lo), (p, max(lo - 1, 0)), (p, p), (p, p + 1), (p, None),
             (0, 0), (page, page - 1), (page - 1, 0), (3 * page + 1, 3 * page)]
    for star in {c[1] for c in cases if c[1] is not None}:
        keys[star] = (keys[star] * 3.0).bfloat16().float()  # long keys: few others point their way by chance
    k_pool = torch.full((n_pages, G, page, dk), float("nan"))
    v_pool = torch.full((n_pages, G, page, dv), float("nan"))
    for j in range(n):
        k_pool[table[0, j // page], :, j % page] = keys[j]
        v_pool[table[0, j // page], :, j % page] = vals[j]
    q = torch.randn(len(cases), H, dk, generator=g) * 0.05
    for t, (_, star) in enumerate(cases):
        for h in range(H):
            if star is None:
                q[t, h] -= 0.5 * keys[:, h // (H // G)].mean(0)  # nothing stands out: the sink matters
            else:
                kk = keys[star, h // (H // G)]
                q[t, h] += 40.0 * kk / kk.norm() ** 2  # its score: 40 * scale
    return dict(n=n, table=table, keys=keys, vals=vals, k_pool=k_pool, v_pool=v_pool, cases=cases,
                q=q.bfloat16().float())


def _check_aimed(c, out, H, G, window, scale, tol):
    for t, (p, star) in enumerate(c["cases"]):
        lo = max(0, p - window + 1) if window else 0
        q1 = c["q"][t].double()[None]
        want = plain.sink_window_attention(
            torch.cat([torch.zeros(p, *q1.shape[1:], dtype=torch.float64), q1]), c["keys"][:p + 1].double(),
            c["vals"][:p + 1].double(), scale, window)[p]
        assert (out[t] - want).abs().max() < tol * max(1.0, want.abs().max().item()), (t, p, star)
        # the case does what it is for: the aimed-at key carries the result iff the query may see it
        s = torch.einsum("hd,jhd->hj", c["q"][t].double(), c["keys"][:p + 1].double().repeat_interleave(H // G, 1)) * scale
        w = torch.exp(s[:, lo:]) / (1 + torch.exp(s[:, lo:]).sum(-1, keepdim=True))
        if star is not None and lo <= star <= p:
            assert w[:, star - lo].min() > 0.5, (t, star)
        elif star is not None:
            # the key is stored but out of sight; had it been seen, it would have carried the result
            s_star = torch.einsum("hd,hd->h", c["q"][t].double(), c["keys"][star].double().repeat_interleave(H // G, 0)) * scale
            seen = torch.exp(s_star) / (1 + torch.exp(s[:, lo:]).sum(-1) + torch.exp(s_star))
            assert seen.min() > 0.5, (t, star)


@pytest.mark.parametrize("pool_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,dk,dv,page,window", [(4, 2, 16, 8, 16, 20), (5, 5, 6, 10, 8, 33), (18, 2, 64, 128, 32, 64),
                                                   (2, 1, 24, 16, 16, 0), (6, 2, 16, 8, 16, 7), (8, 1, 128, 64, 16, 96)])
def test_sink_attention_sees_exactly_the_window(H, G, dk, dv, page, window, pool_dtype):
    from dispec_b200.ops import attention as A
    c = _aimed_attention_case(H, G, dk, dv, page, window, seed=H * dk)
    T = len(c["cases"])
    scale = 0.4
    out = torch.empty((T, H * dv), dtype=pool_dtype, device="cuda:0")
    A.paged_attention_generic(dev(c["q"].reshape(T, -1), pool_dtype), H * dk, dev(c["k_pool"], pool_dtype),
                              dev(c["v_pool"], pool_dtype), c["table"].cuda().expand(T, -1).contiguous(),
                              i32([p for p, _ in c["cases"]]), i32(list(range(T))), out, H, G, dk, window, scale, sink=True)
    out = out.float().cpu().double().view(T, H, dv)
    assert torch.isfinite(out).all()
    _check_aimed(c, out, H, G, window, scale, 2e-4 if pool_dtype == torch.float32 else 0.02)


@pytest.mark.parametrize("H,G,dk,dv,page,window", [(4, 2, 16, 16, 16, 20), (18, 2, 64, 128, 32, 64), (8, 1, 128, 64, 16, 100),
                                                   (12, 2, 128, 128, 16, 0), (6, 2, 32, 16, 8, 7), (5, 5, 48, 32, 16, 33)])
@pytest.mark.parametrize("sink,splits", [(True, 1), (False, 1), (True, 3), (False, 4), (True, 16)])
def test_sink_attention_on_tensor_cores_matches_the_plain_softmax(H, G, dk, dv, page, window, sink, splits):
    """A step of two single tokens and a portion of a prompt whose tiles end in the middle of a key
    tile; every query is aimed at one key: the first of the request, both sides of a page border,
    the first key of its window and the one before it, its own position, the next one (stored,
    invisible), or nothing (the sink takes the weight).  Scattered pages, NaN everywhere else.
    With ``splits`` the single tokens' keys are cut into shares (more shares than key tiles too)
    and merged; the sink must count once."""
    from dispec_b200.ops import attention as A
    g = torch.Generator().manual_seed(H + dk)
    lens, q_lens = [3 * page + 5, 200, 9 * page + 7], [1, 1, 45]
    n_pages = sum(-(-n // page) for n in lens) + 3
    perm = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lens)
    k_pool = torch.full((n_pages, G, page, dk), float("nan"))
    v_pool = torch.full((n_pages, G, page, dv), float("nan"))
    tables, keys, vals, qs, stars = [], [], [], [], []
    aims = ["first", "border-", "border+", "edge_in", "edge_out", "self", "next", None]
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        need = -(-n // page)
        tables.append([perm.pop() for _ in range(need)] + [-1] * (width - need))
        kk = torch.randn(n, G, dk, generator=g).bfloat16().float()
        vv = torch.randn(n, G, dv, generator=g).bfloat16().float()
        qq = torch.randn(ql, H, dk, generator=g) * 0.05
        star = []
        for i in range(ql):
            p = n - ql + i
            lo = max(0, p - window + 1) if window else 0
            a = aims[(i + s) % len(aims)]
            j = {"first": 0, "border-": page - 1, "border+": page, "edge_in": lo, "edge_out": max(lo - 1, 0), "self": p,
                 "next": min(p + 1, n - 1), None: None}[a]
            star.append(j)
        for j in {j for j in star if j is not None}:
            kk[j] = (kk[j] * 3.0).bfloat16().float()
        for i, j in enumerate(star):
            for h in range(H):
                if j is None:
                    qq[i, h] -= 0.5 * kk[:, h // (H // G)].mean(0)
                else:
                    kj = kk[j, h // (H // G)]
                    qq[i, h] += 40.0 * kj / kj.norm() ** 2
        for j in range(n):
            k_pool[tables[-1][j // page], :, j % page] = kk[j]
            v_pool[tables[-1][j // page], :, j % page] = vv[j]
        keys.append(kk); vals.append(vv); qs.append(qq.bfloat16().float()); stars.append(star)
    group = H // G
    assert A.sink_mma_supported(group, dk, dv)
    tpt = A.sink_tokens_per_tile(group, dk, dv)
    tiles = [(s, a) for s, ql in enumerate(q_lens) for a in range(0, ql, tpt)]
    T = sum(q_lens)
    out = torch.full((T, H * dv), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    scale = 0.4
    A.sink_attention_tiles(dev(torch.cat(qs).reshape(T, -1), torch.bfloat16), dev(k_pool, torch.bfloat16),
                           dev(v_pool, torch.bfloat16), i32(tables), i32([0, 1, 2, 2 + q_lens[2]]), i32(lens),
                           i32([s for s, _ in tiles]), i32([a for _, a in tiles]), len(tiles), out, H, G, window, scale, sink,
                           num_single=2, splits=splits)
    out = out.float().cpu().double().view(T, H, dv)
    assert torch.isfinite(out).all()
    at = 0
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        q_full = torch.cat([torch.zeros(n - ql, H, dk), qs[s]]).double()
        if sink:
            want = plain.sink_window_attention(q_full, keys[s].double(), vals[s].double(), scale, window)[n - ql:]
        else:
            want = torch.zeros(ql, H, dv, dtype=torch.float64)
            for i in range(ql):
                p = n - ql + i
                lo = max(0, p - window + 1) if window else 0
                for h in range(H):
                    w = torch.softmax((keys[s][lo:p + 1, h // group].double() @ q_full[p, h]) * scale, dim=0)
                    want[i, h] = w @ vals[s][lo:p + 1, h // group].double()
        err = (out[at:at + ql] - want).abs().amax(dim=(1, 2))
        assert err.max() < 0.03 * max(1.0, want.abs().max().item()), (s, int(err.argmax()), stars[s][int(err.argmax())])
        at += ql
