"""Each part alone, built from a PartSpec with sizes the Llama configurations do not use, against the
plain formula; and a toy mixer with state of its own, defined here, registered, built and stepped
without touching the library's files."""

import numpy as np
import pytest
import torch

from plain_llama import plain_attention, plain_rmsnorm, plain_rope, plain_swiglu_mlp

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx_for(cache, slots, pos0, q_lens, device=DEV):
    """A StepContext and block tables for the given sequences, as Engine.step builds them."""
    from rusty_llama_b200.engine import StepContext

    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    cache.reserve(slots, q_lens)
    tok_seq = sum(([i] * n for i, n in enumerate(q_lens)), [])
    tok_pos = sum((list(range(p, p + n)) for p, n in zip(pos0, q_lens)), [])
    starts = [0] + list(np.cumsum(q_lens))
    width = cache.table_width(slots)
    tables = [torch.from_numpy(cache.block_table(g, slots, width)).to(device) for g in range(len(cache.kv_groups))]
    step = StepContext(
        n_tokens=sum(q_lens), n_seqs=len(slots), max_q_len=max(q_lens), max_kv_len=max(p + n for p, n in zip(pos0, q_lens)),
        plan_kv_len=max(p + n for p, n in zip(pos0, q_lens)), decode_only=all(n == 1 for n in q_lens), slots=list(slots),
        q_lens=list(q_lens), tokens=i32([0] * sum(q_lens)), tok_seq=i32(tok_seq), tok_pos=i32(tok_pos), seq_start=i32(starts),
        seq_pos0=i32(pos0), seq_len=i32([p + n for p, n in zip(pos0, q_lens)]), slot_ids=i32(list(slots)), rows=None,
    )
    return step, tables


def tol(dtype):
    return (2e-5, 1e-6) if dtype == torch.float32 else (1.5e-2, 2.5e-3)


def check(got, ref, dtype):
    if got.dim() == ref.dim() + 1:  # partial sums of a split product: what the next norm would add up
        got = got.float().sum(dim=0)
    got, ref = got.detach().float().cpu().double(), ref.double()
    scale = float(ref.abs().max()) + 1e-9
    mx, mean = tol(dtype)
    err = (got - ref).abs()
    assert float(err.max()) <= mx * scale + 1e-7, f"max error {float(err.max()):.3e} at range {scale:.3e}"
    if dtype != torch.float32:
        assert float(err.mean()) <= mean * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part_adds_what_is_pending(dtype):
    from rusty_llama_b200.parts import NORMS, ResidualStream, Runtime
    from rusty_llama_b200.spec import PartSpec

    rt = Runtime.create(DEV, dtype)
    d = 200
    norm = NORMS.build(PartSpec("rmsnorm", {"size": d, "eps": 2e-6}, "n."), rt)
    assert norm.param_infos()["n.weight"].shape == (d,) and norm.param_infos()["n.weight"].kind == "vector"
    w = 1 + 0.2 * torch.randn(d)
    norm.load({"n.weight": w.to(DEV)})
    x = torch.randn(7, d)
    delta = torch.randn(7, d).to(dtype)
    stream = ResidualStream(x.to(DEV), dtype)
    stream.add(delta.to(DEV))
    out = norm.forward(stream)
    assert stream.pending is None
    total = x + delta.float()
    assert torch.allclose(stream.x.cpu(), total, atol=1e-6)
    check(out, plain_rmsnorm(total.double(), w.double(), 2e-6), dtype)
    # two things added in a row: the first is flushed into the stream
    stream.add(delta.to(DEV))
    stream.add(delta.to(DEV))
    stream.flush()
    assert torch.allclose(stream.x.cpu(), total + 2 * delta.float(), atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from rusty_llama_b200.parts import FEED_FORWARDS, Runtime
    from rusty_llama_b200.spec import PartSpec

    rt = Runtime.create(DEV, dtype)
    d, ff = 72, 200
    mlp = FEED_FORWARDS.build(PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": ff, "activation": "silu"}, "m."), rt)
    w = {"m.gate_proj.weight": torch.randn(ff, d) * 0.1, "m.up_proj.weight": torch.randn(ff, d) * 0.1, "m.down_proj.weight": torch.randn(d, ff) * 0.1}
    w = {k: v.to(dtype) for k, v in w.items()}
    assert {k: v.shape for k, v in mlp.param_infos().items()} == {k: tuple(v.shape) for k, v in w.items()}
    mlp.load({k: v.to(DEV) for k, v in w.items()})
    for T in (1, 9, 100):  # the streaming kernel and the many-row path
        xn = torch.randn(T, d).to(dtype)
        ref = plain_swiglu_mlp(xn.double(), w["m.gate_proj.weight"].double(), w["m.up_proj.weight"].double(), w["m.down_proj.weight"].double())
        check(mlp.forward(xn.to(DEV), None), ref, dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, K, hd, window, interleaved", [(6, 2, 40, 0, False), (3, 3, 24, 50, True), (8, 2, 128, 0, False)])
def test_attention_part_prefill_then_decode(dtype, H, K, hd, window, interleaved):
    """The mixer alone over its own cache: two sequences of unequal lengths whole, then three single tokens each."""
    from rusty_llama_b200.cache import Cache
    from rusty_llama_b200.config import RopeScaling
    from rusty_llama_b200.parts import MIXERS, Runtime
    from rusty_llama_b200.spec import PartSpec

    rt = Runtime.create(DEV, dtype)
    d = 56
    pos = PartSpec("rotary", {"rotary_dim": hd, "theta": 777.0, "scaling": RopeScaling(), "interleaved": interleaved})
    att = MIXERS.build(PartSpec("attention", {"hidden_size": d, "num_heads": H, "num_kv_heads": K, "head_dim": hd, "window": window, "position": pos}, "a."), rt)
    g = torch.Generator().manual_seed(H)
    w = {
        "a.q_proj.weight": torch.randn(H * hd, d, generator=g) * 0.2, "a.k_proj.weight": torch.randn(K * hd, d, generator=g) * 0.2,
        "a.v_proj.weight": torch.randn(K * hd, d, generator=g) * 0.2, "a.o_proj.weight": torch.randn(d, H * hd, generator=g) * 0.2,
    }
    w = {k: v.to(dtype) for k, v in w.items()}
    att.load({k: v.to(DEV) for k, v in w.items()})
    need = att.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.window) == (K, hd, window)
    cache = Cache([(0, need)], 64 * 8, 4, dtype, DEV)
    lens = [70, 9]
    xs = [torch.randn(n + 3, d, generator=g).to(dtype) for n in lens]
    inv = att.position.inv_freq.cpu()

    # the engine keeps q, k, v, the rotated q and k, and the heads' output in the run's type: the
    # reference rounds at the same places, so that what is compared is the arithmetic in between
    rnd = (lambda t: t.to(torch.bfloat16).double()) if dtype == torch.bfloat16 else (lambda t: t)

    def ref_for(x):
        T = x.shape[0]
        xd = x.double()
        q = rnd(xd @ w["a.q_proj.weight"].double().T).view(T, H, hd)
        k = rnd(xd @ w["a.k_proj.weight"].double().T).view(T, K, hd)
        v = rnd(xd @ w["a.v_proj.weight"].double().T).view(T, K, hd)
        q, k = rnd(plain_rope(q, torch.arange(T), inv, interleaved)), rnd(plain_rope(k, torch.arange(T), inv, interleaved))
        return rnd(plain_attention(q, k, v, window).reshape(T, H * hd)) @ w["a.o_proj.weight"].double().T

    refs = [ref_for(x) for x in xs]
    slots = [cache.open_sequence(), cache.open_sequence()]
    step, tables = ctx_for(cache, slots, [0, 0], lens)
    out = att.forward(torch.cat([x[:n] for x, n in zip(xs, lens)]).to(DEV), step, cache.view(0, tables))
    if out.dim() == 3:  # partial sums of a split product: what the next norm would add up
        out = out.float().sum(dim=0)
    cache.commit(slots, lens)
    check(out[: lens[0]], refs[0][: lens[0]], dtype)
    check(out[lens[0] :], refs[1][: lens[1]], dtype)
    for j in range(3):
        step, tables = ctx_for(cache, slots, [n + j for n in lens], [1, 1])
        out = att.forward(torch.stack([x[n + j] for x, n in zip(xs, lens)]).to(DEV), step, cache.view(0, tables))
        if out.dim() == 3:
            out = out.float().sum(dim=0)
        cache.commit(slots, [1, 1])
        check(out[0], refs[0][lens[0] + j], dtype)
        check(out[1], refs[1][lens[1] + j], dtype)


def test_a_layer_can_read_another_layers_cache():
    """A run of the schedule with cache_from: it projects queries only and attends over the keys and
    values the earlier run stored."""
    from rusty_llama_b200.cache import Cache
    from rusty_llama_b200.config import RopeScaling
    from rusty_llama_b200.parts import MIXERS, Runtime
    from rusty_llama_b200.spec import PartSpec

    dtype = torch.float32
    rt = Runtime.create(DEV, dtype)
    d, H, K, hd = 32, 4, 2, 16
    pos = PartSpec("rotary", {"rotary_dim": hd, "theta": 100.0, "scaling": RopeScaling(), "interleaved": False})
    make = lambda p: MIXERS.build(PartSpec("attention", {"hidden_size": d, "num_heads": H, "num_kv_heads": K, "head_dim": hd, "window": 0, "position": pos}, p), rt)
    owner, reader = make("o."), make("r.")
    g = torch.Generator().manual_seed(0)
    ws = {}
    for p in ("o.", "r."):
        ws[p] = {p + "q_proj.weight": torch.randn(H * hd, d, generator=g) * 0.2, p + "k_proj.weight": torch.randn(K * hd, d, generator=g) * 0.2,
                 p + "v_proj.weight": torch.randn(K * hd, d, generator=g) * 0.2, p + "o_proj.weight": torch.randn(d, H * hd, generator=g) * 0.2}
    owner.load({k: v.to(DEV) for k, v in ws["o."].items()})
    reader.load({k: v.to(DEV) for k, v in ws["r."].items()})
    cache = Cache([(0, owner.cache_need())], 64 * 2, 2, dtype, DEV)
    s = cache.open_sequence()
    T = 20
    x1, x2 = torch.randn(T, d, generator=g), torch.randn(T, d, generator=g)
    step, tables = ctx_for(cache, [s], [0], [T])
    owner.forward(x1.to(DEV), step, cache.view(0, tables))
    out = reader.forward(x2.to(DEV), step, cache.view(0, tables), shared_cache=True)
    inv = owner.position.inv_freq.cpu()
    k = plain_rope((x1.double() @ ws["o."]["o.k_proj.weight"].double().T).view(T, K, hd), torch.arange(T), inv, False)
    v = (x1.double() @ ws["o."]["o.v_proj.weight"].double().T).view(T, K, hd)
    q = plain_rope((x2.double() @ ws["r."]["r.q_proj.weight"].double().T).view(T, H, hd), torch.arange(T), inv, False)
    ref = plain_attention(q, k, v).reshape(T, H * hd) @ ws["r."]["r.o_proj.weight"].double().T
    check(out, ref, dtype)


# --------------------------------------------------------------------------- a toy architecture defined here
def register_toy():
    """A mixer with a fixed-size state of its own (a decayed running sum per sequence), a position
    encoding that is not rotary (none) and an architecture that mixes it with attention layer by layer,
    names a layer twice in its schedule and lets one run read another's cache."""
    import rusty_llama_b200 as rl
    from rusty_llama_b200.config import RopeScaling
    from rusty_llama_b200.kernels.linear import linear
    from rusty_llama_b200.parts import MIXERS, Mixer, ParamInfo, StateNeed
    from rusty_llama_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    @MIXERS.register("toy_running_sum", replace=True)
    class RunningSum(Mixer):
        """state <- decay * state + W_in x for each token in order; output W_out state."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.d, self.n, self.decay = spec.params["hidden_size"], spec.params["state_size"], spec.params["decay"]

        def cache_need(self):
            return StateNeed((self.n,), torch.float32)

        def param_infos(self):
            return {self.prefix + "in.weight": ParamInfo((self.n, self.d)), self.prefix + "out.weight": ParamInfo((self.d, self.n))}

        def load(self, tensors):
            self.w_in, self.w_out = tensors[self.prefix + "in.weight"], tensors[self.prefix + "out.weight"]

        def forward(self, xn, step, cache, shared_cache=False):
            u = linear(xn, self.w_in).float()
            idx = step.slot_ids.long()  # device-side, so a replayed graph follows the step's slots
            states = torch.empty_like(u)
            if step.decode_only:
                new = self.decay * cache.state.index_select(0, idx) + u
                cache.state.index_copy_(0, idx, new)
                states = new
            else:
                at = 0
                for i, n in enumerate(step.q_lens):
                    s = cache.state[step.slots[i]].clone()
                    for t in range(n):
                        s = self.decay * s + u[at + t]
                        states[at + t] = s
                    cache.state[step.slots[i]] = s
                    at += n
            return linear(states.to(xn.dtype), self.w_out)

    def parse(d):
        return dict(d)

    def describe(c):
        d = c["width"]
        norm = lambda p: PartSpec("rmsnorm", {"size": d, "eps": c["eps"]}, p)
        ff = lambda p, n: PartSpec("gated_mlp", {"hidden_size": d, "intermediate_size": n, "activation": "silu"}, p)
        att = lambda p, window, position: PartSpec(
            "attention", {"hidden_size": d, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "window": window, "position": position}, p)
        rotary = PartSpec("rotary", {"rotary_dim": 8, "theta": 50.0, "scaling": RopeScaling(), "interleaved": True})
        layers = (
            LayerSpec("prenorm", att("l0.att.", 0, rotary), ff("l0.ff.", 48), {"mixer": norm("l0.n1."), "feed_forward": norm("l0.n2.")}),
            LayerSpec("prenorm", PartSpec("toy_running_sum", {"hidden_size": d, "state_size": 24, "decay": 0.9}, "l1.mix."), ff("l1.ff.", 80),
                      {"mixer": norm("l1.n1."), "feed_forward": norm("l1.n2.")}),
            LayerSpec("prenorm", att("l2.att.", 20, PartSpec("none")), ff("l2.ff.", 48), {"mixer": norm("l2.n1."), "feed_forward": norm("l2.n2.")}),
        )
        schedule = (ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(2), ScheduleEntry(1), ScheduleEntry(0, cache_from=0))
        return ModelSpec("ToyForTests", d, c["vocab"], c["positions"], PartSpec("token_embedding", {"vocab_size": c["vocab"], "hidden_size": d}, "emb."),
                         layers, schedule, norm("final."), PartSpec("linear_head", {"vocab_size": c["vocab"], "hidden_size": d, "tied_to": None}, "head."),
                         stored_dtype="float32")

    rl.register_architecture(rl.Architecture("ToyForTests", parse, describe), replace=True)
    return {"architectures": ["ToyForTests"], "width": 40, "vocab": 97, "positions": 200, "eps": 1e-5}


def toy_plain_logits(cfg, w, tokens):
    """The toy model by its formulas, whole sequence, float64."""
    from plain_llama import plain_silu

    T = len(tokens)
    x = w["emb.weight"].double()[torch.tensor(tokens)]
    pos = torch.arange(T)

    def attention(xn, p, window, rotary, kv=None):
        q = (xn @ w[p + "q_proj.weight"].double().T).view(T, 4, 16)
        if kv is None:
            k = (xn @ w[p + "k_proj.weight"].double().T).view(T, 2, 16)
            v = (xn @ w[p + "v_proj.weight"].double().T).view(T, 2, 16)
        if rotary:
            inv = torch.tensor([50.0 ** (-2 * j / 8) for j in range(4)])
            q = torch.cat([plain_rope(q[..., :8], pos, inv, True), q[..., 8:]], dim=-1)
            if kv is None:
                k = torch.cat([plain_rope(k[..., :8], pos, inv, True), k[..., 8:]], dim=-1)
        if kv is not None:
            k, v = kv
        return plain_attention(q, k, v, window).reshape(T, 64) @ w[p + "o_proj.weight"].double().T, (k, v)

    def running(xn, p):
        u = xn @ w[p + "in.weight"].double().T
        s = torch.zeros(24, dtype=torch.float64)
        out = []
        for t in range(T):
            s = 0.9 * s + u[t]
            out.append(s)
        return torch.stack(out) @ w[p + "out.weight"].double().T

    def ff(xn, p):
        return plain_swiglu_mlp(xn, w[p + "gate_proj.weight"].double(), w[p + "up_proj.weight"].double(), w[p + "down_proj.weight"].double())

    nrm = lambda x, p: plain_rmsnorm(x, w[p + "weight"].double(), cfg["eps"])
    kv0 = None
    for layer, shared in ((0, False), (1, False), (2, False), (1, False), (0, True)):
        p = f"l{layer}."
        xn = nrm(x, p + "n1.")
        if layer == 0:
            a, kv = attention(xn, p + "att.", 0, True, kv0 if shared else None)
            kv0 = kv0 or kv
        elif layer == 2:
            a, _ = attention(xn, p + "att.", 20, False)
        else:
            a = running(xn, p + "mix.")
        x = x + a
        x = x + ff(nrm(x, p + "n2."), p + "ff.")
    return nrm(x, "final.") @ w["head.weight"].double().T


@pytest.mark.parametrize("graphs", [False, True])
def test_toy_architecture_with_a_stateful_mixer(tmp_path, graphs):
    import rusty_llama_b200 as rl
    from conftest import read_weights

    cfg = register_toy()
    model_dir = rl.write_random_model(str(tmp_path / "toy"), cfg, seed=5, std=0.15, norm_jitter=0.1)
    w = read_weights(model_dir)
    assert "l1.mix.in.weight" in w and "l0.att.k_proj.weight" in w
    llm = rl.load(model_dir, dtype="float32", max_tokens=64 * 6, max_seqs=3, use_graphs=graphs)
    cache = llm.engine.cache
    # attention without window, attention with window 20, and the state records (two runs of layer 1) are three groups
    assert len(cache.kv_groups) == 2 and len(cache.state_groups) == 1 and cache.state_groups[0].state.shape == (2, 3, 24)
    rng = np.random.default_rng(2)
    a = rng.integers(0, 97, 100).tolist()
    b = rng.integers(0, 97, 30).tolist()
    ref_a, ref_b = toy_plain_logits(cfg, w, a), toy_plain_logits(cfg, w, b)

    def near(got, ref):
        err = float((got.double().cpu() - ref).abs().max())
        assert err <= 5e-5 * float(ref.abs().max()) + 1e-6, err

    for round_ in range(2):  # the second round runs in reused slots: the state must start from zero again
        sa, sb = llm.open_sequence(), llm.open_sequence()
        out = llm.step([rl.StepEntry(sa, a[:60], list(range(60))), rl.StepEntry(sb, b[:5], list(range(5)))])
        near(out[:60], ref_a[:60])
        near(out[60:], ref_b[:5])
        pa, pb = 60, 5
        while pa < 100:
            entries = [rl.StepEntry(sa, [a[pa]], [0])]
            if pb < 30:
                entries.append(rl.StepEntry(sb, [b[pb]], [0]))
            out = llm.step(entries)
            near(out[0], ref_a[pa])
            if pb < 30:
                near(out[1], ref_b[pb])
                pb += 1
                if pb == 30:
                    llm.close_sequence(sb)
            pa += 1
        llm.close_sequence(sa)
        cache.check_consistent()
    # the window group gave pages back while sequence a grew
    outs = llm.generate([a[:10], b[:3]], max_new_tokens=5, temperature=0.0, stop_token_ids=[])
    assert [len(o) for o in outs] == [5, 5]


# --------------------------------------------------------------------------- a second toy: routing and another position encoding
def register_toy_routed():
    """A feed-forward that routes every token to one of its experts, and a position encoding that is
    not rotary (sinusoids added to queries and keys), both defined here and named layer by layer:
    layer 0 routes over three experts, layer 1 over two of another size and keeps the library's rotary."""
    import rusty_llama_b200 as rl
    from rusty_llama_b200.config import RopeScaling
    from rusty_llama_b200.kernels.linear import linear
    from rusty_llama_b200.parts import FEED_FORWARDS, POSITIONS, FeedForward, ParamInfo, PositionEncoding
    from rusty_llama_b200.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

    @FEED_FORWARDS.register("toy_top1_experts", replace=True)
    class Top1Experts(FeedForward):
        """Router logits r = Wr xn in 32-bit, p = softmax(r); the token goes to expert e = argmax p
        alone and gets p_e * W2_e relu(W1_e xn).  Every expert runs on every token and a mask picks,
        so that shapes never depend on data (a replayed graph stays valid)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.d, self.n, self.E = spec.params["hidden_size"], spec.params["intermediate_size"], spec.params["experts"]

        def param_infos(self):
            infos = {self.prefix + "router.weight": ParamInfo((self.E, self.d))}
            for e in range(self.E):
                infos[f"{self.prefix}experts.{e}.w1.weight"] = ParamInfo((self.n, self.d))
                infos[f"{self.prefix}experts.{e}.w2.weight"] = ParamInfo((self.d, self.n))
            return infos

        def load(self, tensors):
            self.router = tensors[self.prefix + "router.weight"]
            self.w1 = [tensors[f"{self.prefix}experts.{e}.w1.weight"] for e in range(self.E)]
            self.w2 = [tensors[f"{self.prefix}experts.{e}.w2.weight"] for e in range(self.E)]

        def forward(self, xn, step):
            p = torch.softmax(linear(xn, self.router).float(), dim=-1)
            top = p.argmax(dim=-1, keepdim=True)
            gate = torch.zeros_like(p).scatter_(1, top, p.gather(1, top))  # p_e at the chosen expert, 0 elsewhere
            out = torch.zeros_like(xn, dtype=torch.float32)
            for e in range(self.E):
                out += gate[:, e : e + 1] * linear(torch.relu(linear(xn, self.w1[e])), self.w2[e]).float()
            return out.to(xn.dtype)

    @POSITIONS.register("toy_added_sinusoid", replace=True)
    class AddedSinusoid(PositionEncoding):
        """q and k of every head get table[pos] added, table[pos, j] = amp * sin(pos / base^(j / hd) + j)."""

        def __init__(self, spec, runtime):
            super().__init__(spec, runtime)
            self.base, self.amp = float(spec.params["base"]), float(spec.params["amplitude"])

        def rotate(self, q, k, step):
            hd = q.shape[-1]
            j = torch.arange(hd, device=q.device, dtype=torch.float32)
            ang = step.tok_pos.float()[:, None] / (self.base ** (j / hd))[None, :] + j[None, :]
            add = (self.amp * torch.sin(ang)).to(q.dtype)[:, None, :]
            q += add
            k += add

    def describe(c):
        d = c["width"]
        norm = lambda p: PartSpec("rmsnorm", {"size": d, "eps": c["eps"]}, p)
        experts = lambda p, n, E: PartSpec("toy_top1_experts", {"hidden_size": d, "intermediate_size": n, "experts": E}, p)
        att = lambda p, position: PartSpec(
            "attention", {"hidden_size": d, "num_heads": 3, "num_kv_heads": 1, "head_dim": 24, "window": 0, "position": position}, p)
        layers = (
            LayerSpec("prenorm", att("l0.att.", PartSpec("toy_added_sinusoid", {"base": 30.0, "amplitude": 0.5})), experts("l0.moe.", 56, 3),
                      {"mixer": norm("l0.n1."), "feed_forward": norm("l0.n2.")}),
            LayerSpec("prenorm", att("l1.att.", PartSpec("rotary", {"rotary_dim": 24, "theta": 80.0, "scaling": RopeScaling(), "interleaved": False})),
                      experts("l1.moe.", 40, 2), {"mixer": norm("l1.n1."), "feed_forward": norm("l1.n2.")}),
        )
        return ModelSpec("ToyRoutedForTests", d, c["vocab"], c["positions"], PartSpec("token_embedding", {"vocab_size": c["vocab"], "hidden_size": d}, "emb."),
                         layers, (ScheduleEntry(0), ScheduleEntry(1)), norm("final."),
                         PartSpec("linear_head", {"vocab_size": c["vocab"], "hidden_size": d, "tied_to": "emb.weight"}, "head."), stored_dtype="float32")

    rl.register_architecture(rl.Architecture("ToyRoutedForTests", dict, describe), replace=True)
    return {"architectures": ["ToyRoutedForTests"], "width": 48, "vocab": 61, "positions": 150, "eps": 1e-6}


def toy_routed_plain_logits(cfg, w, tokens):
    """The second toy model by its formulas, whole sequence, float64; also returns the experts chosen."""
    T = len(tokens)
    x = w["emb.weight"].double()[torch.tensor(tokens)]
    pos = torch.arange(T)
    chosen = []
    for layer in (0, 1):
        p = f"l{layer}."
        xn = plain_rmsnorm(x, w[p + "n1.weight"].double(), cfg["eps"])
        q = (xn @ w[p + "att.q_proj.weight"].double().T).view(T, 3, 24)
        k = (xn @ w[p + "att.k_proj.weight"].double().T).view(T, 1, 24)
        v = (xn @ w[p + "att.v_proj.weight"].double().T).view(T, 1, 24)
        if layer == 0:
            j = torch.arange(24, dtype=torch.float64)
            add = 0.5 * torch.sin(pos.double()[:, None] / (30.0 ** (j / 24))[None, :] + j[None, :])
            q, k = q + add[:, None, :], k + add[:, None, :]
        else:
            inv = torch.tensor([80.0 ** (-2 * i / 24) for i in range(12)])
            q, k = plain_rope(q, pos, inv, False), plain_rope(k, pos, inv, False)
        x = x + plain_attention(q, k, v, 0).reshape(T, 72) @ w[p + "att.o_proj.weight"].double().T
        xn = plain_rmsnorm(x, w[p + "n2.weight"].double(), cfg["eps"])
        prob = torch.softmax(xn @ w[p + "moe.router.weight"].double().T, dim=-1)
        top = prob.argmax(dim=-1)
        chosen.append(top)
        ff = torch.zeros_like(x)
        for t in range(T):
            e = int(top[t])
            h = torch.relu(xn[t] @ w[f"{p}moe.experts.{e}.w1.weight"].double().T)
            ff[t] = prob[t, e] * (h @ w[f"{p}moe.experts.{e}.w2.weight"].double().T)
        x = x + ff
    return plain_rmsnorm(x, w["final.weight"].double(), cfg["eps"]) @ w["emb.weight"].double().T, chosen


@pytest.mark.parametrize("graphs", [False, True])
def test_toy_architecture_with_routed_experts_and_added_positions(tmp_path, graphs):
    """A feed-forward with routing and a position encoding of another kind, registered from here,
    built from a configuration, loaded from a model folder and stepped (prompts of unequal lengths,
    then token by token, twice in reused slots) without a change to the library's files."""
    import rusty_llama_b200 as rl
    from conftest import read_weights

    cfg = register_toy_routed()
    model_dir = rl.write_random_model(str(tmp_path / "toy_routed"), cfg, seed=11, std=0.25, norm_jitter=0.1)
    w = read_weights(model_dir)
    assert "l0.moe.experts.2.w1.weight" in w and "l1.moe.router.weight" in w and "head.weight" not in w
    llm = rl.load(model_dir, dtype="float32", max_tokens=64 * 5, max_seqs=2, use_graphs=graphs)
    rng = np.random.default_rng(8)
    a, b = rng.integers(0, 61, 90).tolist(), rng.integers(0, 61, 21).tolist()
    (ref_a, chosen_a), (ref_b, _) = toy_routed_plain_logits(cfg, w, a), toy_routed_plain_logits(cfg, w, b)
    # the routing is exercised: every expert of both layers is chosen by some token
    assert set(chosen_a[0].tolist()) == {0, 1, 2} and set(chosen_a[1].tolist()) == {0, 1}

    def near(got, ref):
        err = float((got.double().cpu() - ref).abs().max())
        assert err <= 5e-5 * float(ref.abs().max()) + 1e-6, err

    for round_ in range(2):
        sa, sb = llm.open_sequence(), llm.open_sequence()
        out = llm.step([rl.StepEntry(sa, a[:50], list(range(50))), rl.StepEntry(sb, b[:4], list(range(4)))])
        near(out[:50], ref_a[:50])
        near(out[50:], ref_b[:4])
        pa, pb = 50, 4
        while pa < 90:
            entries = [rl.StepEntry(sa, [a[pa]], [0])]
            if pb < 21:
                entries.append(rl.StepEntry(sb, [b[pb]], [0]))
            out = llm.step(entries)
            near(out[0], ref_a[pa])
            if pb < 21:
                near(out[1], ref_b[pb])
                pb += 1
                if pb == 21:
                    llm.close_sequence(sb)
            pa += 1
        llm.close_sequence(sa)
        llm.engine.cache.check_consistent()
    outs = llm.generate([a[:10], b[:3]], max_new_tokens=5, temperature=0.0, stop_token_ids=[])
    assert [len(o) for o in outs] == [5, 5]
