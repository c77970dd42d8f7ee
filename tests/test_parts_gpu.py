"""Each part of a layer alone against the plain implementation's function for it, and a toy mixer
with state of its own that is registered, built and stepped without touching the framework."""
import pytest
import torch

import plain_qwen2 as plain
from tiny import make_folder, prompt

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _ctx(q_lens, q_starts, dtype):
    from ginfer_b200.parts import StepContext
    B, T = len(q_lens), sum(q_lens)
    cu = [0]
    for n in q_lens:
        cu.append(cu[-1] + n)
    pos = torch.cat([torch.arange(s, s + n) for s, n in zip(q_starts, q_lens)])
    seq = torch.cat([torch.full((n,), b) for b, n in enumerate(q_lens)])
    i32 = lambda t: torch.as_tensor(t, dtype=torch.int32, device=DEV)
    return StepContext(
        num_tokens=T, num_seqs=B, dtype=dtype, device=DEV, token_ids=i32([0] * T),
        positions=i32(pos), seq_of_token=i32(seq), cu_seqlens_q=i32(cu),
        kv_lens=i32([s + n for s, n in zip(q_starts, q_lens)]), slot_ids=i32(list(range(B))),
        logit_rows=i32([]), q_lens_host=list(q_lens), q_starts_host=list(q_starts),
        slot_ids_host=list(range(B)), max_q_len=max(q_lens),
        max_kv_len=max(s + n for s, n in zip(q_starts, q_lens)), decode_only=max(q_lens) == 1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from ginfer_b200.parts import PartSpec, make_part
    H, eps = 200, 3e-4
    norm = make_part("norm", PartSpec("rmsnorm", dict(size=H, eps=eps, weight_name="g")))
    assert [(s.name, s.shape, s.role) for s in norm.tensor_specs()] == [("g", (H,), "norm")]
    g = (1 + 0.3 * torch.randn(H)).to(DEV)
    norm.load({"g": g}, dtype, DEV)
    x = torch.randn(9, H, device=DEV)
    d = torch.randn(9, H, device=DEV).to(dtype)
    s, n = norm.forward(x, d)
    want = plain.rms_norm(x.double() + d.double(), g.double(), eps)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(n.double(), want, **tol)
    torch.testing.assert_close(s.double(), x.double() + d.double(), atol=1e-6, rtol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from ginfer_b200.parts import PartSpec, make_part
    H, I = 96, 224
    ffn = make_part("feed_forward", PartSpec("swiglu", dict(hidden_size=H, intermediate_size=I,
                                                            prefix="mlp")))
    names = {s.name: s.shape for s in ffn.tensor_specs()}
    assert names == {"mlp.gate_proj.weight": (I, H), "mlp.up_proj.weight": (I, H),
                     "mlp.down_proj.weight": (H, I)}
    w = {k: (torch.randn(*shape) * 0.1).to(dtype).to(DEV) for k, shape in names.items()}
    ffn.load(w, dtype, DEV)
    x = torch.randn(11, H).to(dtype).to(DEV)
    got = ffn.forward(x, _ctx([11], [0], dtype))
    if dtype == torch.bfloat16:
        plain.Stored.bf16()
    try:
        want = plain.swiglu(x.double().cpu(), w["mlp.gate_proj.weight"].double().cpu(),
                            w["mlp.up_proj.weight"].double().cpu(),
                            w["mlp.down_proj.weight"].double().cpu())
    finally:
        plain.Stored.exact()
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(got.double().cpu(), want, **tol)


def test_rotary_part_table():
    from ginfer_b200.parts import PartSpec, make_part
    hd, theta, n = 48, 50000.0, 300
    rot = make_part("position", PartSpec("rotary", dict(head_dim=hd, theta=theta,
                                                        max_positions=n)))
    rot.load({}, torch.float32, DEV)
    table, dim = rot.rotary_table()
    assert dim == hd and table.shape == (n, hd) and table.dtype == torch.float32
    cos, sin = plain.rotary_cos_sin(torch.arange(n), hd, theta)
    torch.testing.assert_close(table[:, :hd // 2].double().cpu(), cos, atol=1e-7, rtol=0)
    torch.testing.assert_close(table[:, hd // 2:].double().cpu(), sin, atol=1e-7, rtol=0)
    assert make_part("position", PartSpec("none")).rotary_table() == (None, 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [0, 21])
def test_attention_part_over_its_cache(dtype, window):
    """The mixer alone: a prompt in two portions, then single tokens, against plain attention
    over the whole sequence."""
    from ginfer_b200.parts import PagedKVBinding, PartSpec, make_part
    H, nh, nkv, hd, P = 80, 6, 2, 32, 8
    attn = make_part("mixer", PartSpec("attention", dict(
        hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd, window=window,
        position=PartSpec("rotary", dict(head_dim=hd, theta=1e4, max_positions=256)))))
    specs = {s.name: s for s in attn.tensor_specs()}
    assert specs["self_attn.k_proj.weight"].shape == (nkv * hd, H)
    assert specs["self_attn.q_proj.bias"].role == "bias" and "self_attn.o_proj.bias" not in specs
    g = torch.Generator().manual_seed(1)
    w = {k: (torch.randn(*s.shape, generator=g) * (0.4 if "q_proj" in k or "k_proj" in k
                                                    else 0.1)).to(dtype).to(DEV)
         for k, s in specs.items()}
    attn.load(w, dtype, DEV)
    cs = attn.cache_spec()
    assert (cs.num_kv_heads, cs.head_dim, cs.window) == (nkv, hd, window)
    T = 75
    x = torch.randn(T, H, generator=g).to(dtype).to(DEV)
    pages = torch.zeros(2, 16, P, nkv, hd, dtype=dtype, device=DEV)
    perm = torch.randperm(16, generator=g).to(torch.int32)
    table = perm[:10].reshape(1, 10).to(DEV)
    outs, at = [], 0
    for n in [40, 23, 1, 1, 1, 9]:
        ctx = _ctx([n], [at], dtype)
        pos = torch.arange(at, at + n)
        slots = (perm[(pos // P).long()] * P + pos % P).to(torch.int32).to(DEV)
        outs.append(attn.forward(x[at:at + n].contiguous(), ctx,
                                 PagedKVBinding(pages, table, slots, P, window, True)))
        at += n
    got = torch.cat(outs)
    if dtype == torch.bfloat16:
        plain.Stored.bf16()
    try:
        cw = {("model.layers.0." + k): v.double().cpu() for k, v in w.items()}
        cfg = dict(num_attention_heads=nh, num_key_value_heads=nkv, head_dim=hd, hidden_size=H,
                   rope_theta=1e4)
        q, k, v = plain.project_qkv(x.double().cpu(), cw, "model.layers.0", cfg, torch.arange(T))
        o = plain.gqa_attention(q, k, v, window)
        want = plain.linear(o.reshape(T, -1), cw["model.layers.0.self_attn.o_proj.weight"])
    finally:
        plain.Stored.exact()
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(got.double().cpu(), want, **tol)


def test_embedding_and_head_parts():
    from ginfer_b200.parts import PartSpec, make_part
    V, H = 301, 80
    emb = make_part("embedding", PartSpec("token", dict(vocab_size=V, hidden_size=H, name="E")))
    head = make_part("head", PartSpec("linear", dict(vocab_size=V, hidden_size=H, tied_to="E")))
    assert head.tensor_specs() == []                       # tied: no tensor of its own
    E = torch.randn(V, H).to(torch.bfloat16).to(DEV)
    emb.load({"E": E}, torch.bfloat16, DEV)
    head.load({"E": E}, torch.bfloat16, DEV)
    ids = torch.tensor([5, 300, 0], dtype=torch.int32, device=DEV)
    ctx = _ctx([3], [0], torch.bfloat16)
    assert torch.equal(emb.forward(ids, ctx), E[ids.long()])
    x = torch.randn(4, H).to(torch.bfloat16).to(DEV)
    logits = head.forward(x, ctx)
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.double(), x.double() @ E.double().t(), atol=1e-3, rtol=1e-3)


# ----------------------------------------------------------------------------- a toy architecture
def test_a_toy_mixer_with_state_of_its_own_registers_builds_and_steps(tmp_path):
    """Defined here, not in the framework: a mixer that keeps, per request, the running sum of
    its inputs and the token count (state of fixed size in a slot), and mixes each token with the
    mean of everything before it.  An architecture that alternates it with attention layers is
    registered, gets random weights through the framework's own writer, is loaded and stepped in
    portions and mixed batches; the result equals a whole-sequence computation."""
    from ginfer_b200.config import register_architecture
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.parts import (LayerSpec, Mixer, ModelPlan, PartSpec, RunEntry, StateSpec,
                                   TensorSpec, register_mixer)
    from ginfer_b200.weights import write_random_model

    class RunningMean(Mixer):
        def __init__(self, hidden_size, prefix="mean"):
            self.h, self.prefix = hidden_size, prefix

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.scale", (self.h,), "norm")]

        def load(self, tensors, dtype, device):
            self.scale = tensors[f"{self.prefix}.scale"].float()

        def cache_spec(self):
            return StateSpec((self.h + 1,), torch.float32)      # the sum and the count

        def forward(self, x, ctx, cache):
            if ctx.decode_only:
                # one token a request: device indices only, so that the step can be captured in
                # a CUDA graph and replayed for other requests and slots
                slots = ctx.slot_ids.long()
                st = cache.state[slots]
                sums = st[:, :self.h] + x.float()
                counts = st[:, self.h] + 1
                if cache.write:
                    cache.state[slots] = torch.cat([sums, counts[:, None]], dim=1)
                return (sums / counts[:, None] * self.scale).to(x.dtype)
            out = torch.empty_like(x)
            at = 0
            for b, n in enumerate(ctx.q_lens_host):             # plain torch: a toy, not a kernel
                st = cache.state[ctx.slot_ids_host[b]]
                xs = x[at:at + n].float()
                sums = st[:self.h] + torch.cumsum(xs, 0)
                counts = st[self.h] + torch.arange(1, n + 1, device=x.device)
                out[at:at + n] = (sums / counts[:, None] * self.scale).to(x.dtype)
                if cache.write:
                    st[:self.h] = sums[-1]
                    st[self.h] = counts[-1]
                at += n
            return out

    register_mixer("running_mean", RunningMean)

    class ToyConfig:
        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d)

        torch_dtype = "float32"

    def toy_plan(cfg):
        d = cfg.d
        H, V = d["hidden_size"], d["vocab_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=1e-5, weight_name=name))
        ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=d["intermediate_size"]))
        attn = PartSpec("attention", dict(
            hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16,
            position=PartSpec("rotary", dict(head_dim=16, theta=1e4, max_positions=256))))
        layers = (
            LayerSpec("toy.0", PartSpec("running_mean", dict(hidden_size=H)), ffn, norm("n1"),
                      norm("n2")),
            LayerSpec("toy.1", attn, ffn, norm("n1"), norm("n2")),
        )
        # the run list names layer 0 twice (two caches) and layer 1 once
        run = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2))
        return ModelPlan(hidden_size=H, vocab_size=V, max_positions=256,
                         embedding=PartSpec("token", dict(vocab_size=V, hidden_size=H, name="emb")),
                         layers=layers, run=run, final_norm=norm("final"),
                         head=PartSpec("linear", dict(vocab_size=V, hidden_size=H, tied_to="emb")))

    register_architecture("ToyRunningMeanLM", ToyConfig, toy_plan)
    cfg = {"architectures": ["ToyRunningMeanLM"], "hidden_size": 64, "vocab_size": 120,
           "intermediate_size": 96}
    d = str(tmp_path / "toy")
    write_random_model(d, cfg, seed=3, storage_dtype="float32")
    model, _ = load_model(d, "float32")
    specs = model.cache_specs()
    assert isinstance(specs[0], StateSpec) and isinstance(specs[2], StateSpec)

    def runner():
        return ModelRunner(model, page_size=8, max_num_seqs=3, max_seq_len=128, num_pages=24)

    reqs = {"a": prompt(50, 120, 1), "b": prompt(31, 120, 2), "c": prompt(17, 120, 3)}
    whole = {}
    r = runner()
    for rid, toks in reqs.items():
        whole[rid] = r.step([StepEntry(rid, toks, list(range(len(toks))))]).cpu()
        r.end(rid)
    # the same in portions, mixed, with slots reused by a later request
    r = runner()
    got = {k: [] for k in reqs}
    at = {k: 0 for k in reqs}
    plan = [[("a", 20), ("b", 5)], [("a", 1), ("b", 26)], [("a", 29), ("c", 2)], [("c", 15)]]
    for step in plan:
        entries = []
        for rid, n in step:
            entries.append(StepEntry(rid, reqs[rid][at[rid]:at[rid] + n], list(range(n))))
            at[rid] += n
        out = r.step(entries).cpu()
        o = 0
        for rid, n in step:
            got[rid].append(out[o:o + n])
            o += n
        for rid, _ in step:
            if at[rid] == len(reqs[rid]):
                r.end(rid)
    for rid in reqs:
        torch.testing.assert_close(torch.cat(got[rid]), whole[rid], atol=2e-5, rtol=1e-4)
    # decoding from CUDA graphs: models with state in slots warm up and replay like the others
    # (the rows that pad a batch up to a graph's size use the slot that no request owns)
    r = ModelRunner(model, page_size=8, max_num_seqs=12, max_seq_len=128, num_pages=24,
                    enforce_eager=False)
    r.warmup()
    names = list(reqs) + ["d", "e", "f", "g", "h", "i"]
    toks = {**reqs, **{k: prompt(12 + i, 120, 10 + i) for i, k in enumerate(names[3:])}}
    alone = {}
    for k in names[3:]:
        r0 = runner()
        alone[k] = r0.step([StepEntry(k, toks[k], list(range(len(toks[k]))))]).cpu()
    alone.update(whole)
    r.step([StepEntry(k, toks[k][:8], []) for k in names])          # nine requests: a graph of 16
    for i in range(8, 12):
        out = r.step([StepEntry(k, [toks[k][i]], [0]) for k in names]).cpu()
        for j, k in enumerate(names):
            torch.testing.assert_close(out[j], alone[k][i], atol=2e-5, rtol=1e-4)
    assert r.graph_launches > 0 and any(k[0] == 16 for k in r._graphs)
    # the state really is used: the mean mixer sees earlier tokens
    other = list(reqs["a"])
    other[0] = (other[0] + 1) % 120
    r2 = runner()
    changed = r2.step([StepEntry("a", other, [49])]).cpu()
    assert not torch.allclose(changed[0], whole["a"][49], atol=1e-4)


def test_a_toy_mixer_that_caches_one_vector_a_token_registers_builds_and_steps(tmp_path):
    """Defined here, not in the framework: a mixer whose paged cache holds ONE vector of 24
    channels per token (neither keys and values nor heads: ``PagedKVSpec(planes=((1, 24),))``)
    and whose output mixes each token with the mean of the cached vectors of the last ``window``
    positions.  The cache manager, the storage and the step function take it as they take
    attention: pages, block table, slot mapping, a window that gives pages back."""
    from ginfer_b200.config import register_architecture
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.parts import (LayerSpec, Mixer, ModelPlan, PagedKVSpec, PartSpec,
                                   TensorSpec, register_mixer, sequential_run)
    from ginfer_b200.weights import write_random_model
    WIDTH = 24

    class LatentMean(Mixer):
        def __init__(self, hidden_size, window, prefix="latent"):
            self.h, self.window, self.prefix = hidden_size, window, prefix

        def tensor_specs(self):
            return [TensorSpec(f"{self.prefix}.down.weight", (WIDTH, self.h)),
                    TensorSpec(f"{self.prefix}.up.weight", (self.h, WIDTH))]

        def load(self, tensors, dtype, device):
            self.down = tensors[f"{self.prefix}.down.weight"].float()
            self.up = tensors[f"{self.prefix}.up.weight"].float()

        def cache_spec(self):
            return PagedKVSpec(1, WIDTH, self.window, planes=((1, WIDTH),))

        def forward(self, x, ctx, cache):
            (plane,) = cache.pages                              # [pages, page, 1, WIDTH]
            flat = plane.view(-1, WIDTH)
            lat = x.float() @ self.down.t()
            if cache.write:
                flat[cache.slot_mapping.long()] = lat.to(flat.dtype)
            out = torch.empty_like(x)
            at = 0
            for b, (n, start) in enumerate(zip(ctx.q_lens_host, ctx.q_starts_host)):
                table = cache.block_table[b].long()
                for i in range(n):                              # plain torch: a toy, not a kernel
                    p = start + i
                    pos = torch.arange(max(0, p - self.window + 1), p + 1, device=x.device)
                    rows = table[pos // cache.page_size] * cache.page_size + pos % cache.page_size
                    mean = flat[rows].float().mean(0)
                    out[at + i] = ((lat[at + i] + mean) @ self.up.t()).to(x.dtype)
                at += n
            return out

    register_mixer("latent_mean", LatentMean)

    class ToyConfig:
        torch_dtype = "float32"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d)

    def toy_plan(cfg):
        H, V = cfg.d["hidden_size"], cfg.d["vocab_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=1e-5, weight_name=name))
        ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=96))
        attn = PartSpec("attention", dict(
            hidden_size=H, num_heads=4, num_kv_heads=2, head_dim=16,
            position=PartSpec("rotary", dict(head_dim=16, theta=1e4, max_positions=256))))
        layers = (LayerSpec("toy.0", PartSpec("latent_mean", dict(hidden_size=H, window=21)), ffn,
                            norm("n1"), norm("n2")),
                  LayerSpec("toy.1", attn, ffn, norm("n1"), norm("n2")))
        return ModelPlan(hidden_size=H, vocab_size=V, max_positions=256,
                         embedding=PartSpec("token", dict(vocab_size=V, hidden_size=H, name="emb")),
                         layers=layers, run=sequential_run(2), final_norm=norm("final"),
                         head=PartSpec("linear", dict(vocab_size=V, hidden_size=H, tied_to="emb")))

    register_architecture("ToyLatentLM", ToyConfig, toy_plan)
    cfg = {"architectures": ["ToyLatentLM"], "hidden_size": 64, "vocab_size": 120}
    d = str(tmp_path / "latent")
    write_random_model(d, cfg, seed=4, storage_dtype="float32")
    model, _ = load_model(d, "float32")
    r = ModelRunner(model, page_size=8, max_num_seqs=2, max_seq_len=128, num_pages=32,
                    max_num_batched_tokens=96)
    # two cache groups: the latent one (a plane of its own, windowed: few pages) and attention's
    kinds = sorted((g.planes, g.stacked, g.window) for g in r.groups)
    assert kinds == [(((1, WIDTH),), False, 21), (((2, 16), (2, 16)), True, 0)]
    latent = next(i for i, g in enumerate(r.groups) if not g.stacked)
    # 2 requests keep 3 + 2 pages of their windows live, a step brings at most 12 pages
    assert r.cache.pools[latent].num_pages == 22 and r.cache.pools[1 - latent].num_pages == 32
    assert isinstance(r.storage.pages_of(0), tuple) and r.storage.pages_of(0)[0].shape[1:] == \
        (8, 1, WIDTH)
    toks = prompt(90, 120, 5)
    whole = r.step([StepEntry("w", toks, list(range(90)))]).cpu()
    r.end("w")
    got, at = [], 0
    for n in (30, 1, 17, 2, 40):                                # the window passes pages: given back
        got.append(r.step([StepEntry("p", toks[at:at + n], list(range(n)))]).cpu())
        at += n
        r.cache.check()
    torch.testing.assert_close(torch.cat(got), whole, atol=2e-5, rtol=1e-4)
    moved = list(toks)
    moved[70] = (moved[70] + 1) % 120                           # within the window of token 89
    r.end("p")
    assert not torch.allclose(r.step([StepEntry("m", moved, [89])]).cpu()[0], whole[89], atol=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding_register_and_step(tmp_path, dtype):
    """Two more parts defined here, not in the framework.  A feed-forward with routing: a router
    scores three small experts in 32-bit, each token goes through its best expert, scaled by the
    router's softmax weight.  A position encoding with code of its own: q and k are scaled, channel
    by channel, by a cosine of the position.  One layer uses both, the other the framework's own
    parts; the layers of the model therefore differ in mixer options and in feed-forward.  Whole
    prompts, portions and decoding one by one agree; moving a token changes later logits."""
    from ginfer_b200 import ops
    from ginfer_b200.config import register_architecture
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import load_model
    from ginfer_b200.parts import (FeedForward, LayerSpec, ModelPlan, PartSpec, PositionEncoding,
                                   TensorSpec, register_feed_forward, register_position,
                                   sequential_run)
    from ginfer_b200.weights import write_random_model

    class RoutedFF(FeedForward):
        def __init__(self, hidden_size, expert_size, num_experts, prefix="moe"):
            self.h, self.e, self.n, self.prefix = hidden_size, expert_size, num_experts, prefix

        def tensor_specs(self):
            out = [TensorSpec(f"{self.prefix}.router.weight", (self.n, self.h))]
            for i in range(self.n):
                out += [TensorSpec(f"{self.prefix}.experts.{i}.up.weight", (self.e, self.h)),
                        TensorSpec(f"{self.prefix}.experts.{i}.down.weight", (self.h, self.e))]
            return out

        def load(self, tensors, dtype, device):
            self.router = tensors[f"{self.prefix}.router.weight"].float()
            self.up = [ops.Linear(tensors[f"{self.prefix}.experts.{i}.up.weight"])
                       for i in range(self.n)]
            self.down = [ops.Linear(tensors[f"{self.prefix}.experts.{i}.down.weight"])
                         for i in range(self.n)]

        def forward(self, x, ctx):
            scores = torch.softmax(x.float() @ self.router.t(), dim=-1)   # router in 32-bit
            weight, choice = scores.max(dim=-1)
            out = torch.zeros_like(x)
            for i in range(self.n):                                       # plain torch: a toy
                rows = torch.nonzero(choice == i).flatten()
                if rows.numel():
                    y = self.down[i](torch.relu(self.up[i](x[rows].contiguous())))
                    out[rows] = (y.float() * weight[rows, None]).to(x.dtype)
            return out

    class CosineScale(PositionEncoding):
        def __init__(self, head_dim, period):
            self.freq = torch.arange(1, head_dim + 1, dtype=torch.float32) / (head_dim * period)

        def load(self, tensors, dtype, device):
            self.freq = self.freq.to(device)

        def apply(self, q, k, ctx):                    # rotary_table() stays None: code of its own
            f = torch.cos(ctx.positions.float()[:, None] * self.freq)[:, None, :]
            q.copy_((q.float() * f).to(q.dtype))
            k.copy_((k.float() * f).to(k.dtype))

    register_feed_forward("toy_routed", RoutedFF)
    register_position("toy_cosine_scale", CosineScale)

    class ToyConfig:
        torch_dtype = "float32"

        def __init__(self, d):
            self.d = dict(d)

        @classmethod
        def from_dict(cls, d):
            return cls(d)

        def to_dict(self):
            return dict(self.d)

    def toy_plan(cfg):
        H, V = cfg.d["hidden_size"], cfg.d["vocab_size"]
        norm = lambda name: PartSpec("rmsnorm", dict(size=H, eps=2e-5, weight_name=name))
        attn = lambda pos, heads, kv: PartSpec("attention", dict(
            hidden_size=H, num_heads=heads, num_kv_heads=kv, head_dim=16, position=pos))
        rotary = PartSpec("rotary", dict(head_dim=16, theta=1e4, max_positions=256))
        layers = (
            LayerSpec("l0", attn(PartSpec("toy_cosine_scale", dict(head_dim=16, period=7.0)), 4, 4),
                      PartSpec("toy_routed", dict(hidden_size=H, expert_size=40, num_experts=3)),
                      norm("n1"), norm("n2")),
            LayerSpec("l1", attn(rotary, 6, 2),
                      PartSpec("swiglu", dict(hidden_size=H, intermediate_size=104)),
                      norm("n1"), norm("n2")),
        )
        return ModelPlan(hidden_size=H, vocab_size=V, max_positions=256,
                         embedding=PartSpec("token", dict(vocab_size=V, hidden_size=H, name="emb")),
                         layers=layers, run=sequential_run(2), final_norm=norm("final"),
                         head=PartSpec("linear", dict(vocab_size=V, hidden_size=H, name="head")))

    register_architecture("ToyRoutedLM", ToyConfig, toy_plan)
    cfg = {"architectures": ["ToyRoutedLM"], "hidden_size": 48, "vocab_size": 90}
    d = str(tmp_path / "toy_routed")
    write_random_model(d, cfg, seed=4, storage_dtype=dtype)
    model, _ = load_model(d, dtype)

    def runner():
        return ModelRunner(model, page_size=8, max_num_seqs=2, max_seq_len=128, num_pages=20)

    toks = prompt(60, 90, 9)
    r = runner()
    whole = r.step([StepEntry("a", toks, list(range(60)))]).cpu()
    r = runner()
    parts, at = [], 0
    for n in (17, 2, 30, 1, 1, 1, 8):                  # portions, then tokens one by one
        parts.append(r.step([StepEntry("a", toks[at:at + n], list(range(n)))]).cpu())
        at += n
    got = torch.cat(parts)
    if dtype == "float32":
        torch.testing.assert_close(got, whole, atol=2e-5, rtol=1e-4)
    else:
        # bfloat16: a token near a tie between experts may flip; compare where routing is stable
        close = (got - whole).abs().amax(dim=-1) <= 2.0 ** -6 * whole.abs().max()
        assert close.float().mean() >= 0.9, f"only {int(close.sum())} of 60 positions agree"
    other = list(toks)
    other[3] = (other[3] + 1) % 90
    changed = runner().step([StepEntry("a", other, [59])]).cpu()
    assert not torch.allclose(changed[0], whole[59], atol=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_list_names_a_layer_twice_and_shares_a_cache(tmp_path, dtype):
    """A Qwen2 folder run under another plan: layer 0 runs twice (second time with a cache of its
    own) and the last run of layer 1 reads the cache layer 1 wrote; compared with plain."""
    import replay
    from ginfer_b200.config.registry import resolve_architecture
    from ginfer_b200.engine import ModelRunner, StepEntry
    from ginfer_b200.engine.loading import parse_dtype
    from ginfer_b200.parts import DecoderModel, ModelPlan, RunEntry
    from ginfer_b200.weights import load_weights
    import dataclasses
    d = make_folder(tmp_path, "A", seed=8, storage=dtype)
    arch = resolve_architecture(plain.read_model_folder(d)[0])
    cfg = arch.config_cls.from_json_file(d)
    base = arch.build_plan(cfg)
    run = (RunEntry(0, 0), RunEntry(1, 1), RunEntry(0, 2), RunEntry(1, 1, write_cache=False))
    model = DecoderModel(dataclasses.replace(base, run=run))
    load_weights(model, d, parse_dtype(dtype), DEV)
    r = ModelRunner(model, page_size=16, max_num_seqs=2, max_seq_len=128, num_pages=16)
    toks = prompt(70, cfg.vocab_size, 5)
    rows = []
    at = 0
    for n in [33, 2, 1, 1, 30, 3]:
        rows.append(r.step([StepEntry("x", toks[at:at + n], list(range(n)))]).cpu())
        at += n
    got = torch.cat(rows).double().numpy()
    pcfg, w = plain.read_model_folder(d)
    if dtype == "bfloat16":
        plain.Stored.bf16()
    try:
        want = plain.forward(w, pcfg, toks, run=[(0, 0, True), (1, 1, True), (0, 2, True),
                                                 (1, 1, False)]).numpy()
    finally:
        plain.Stored.exact()
    import numpy as np
    atol, rtol = replay.tolerances(dtype, float(np.abs(want).max()))
    assert np.all(np.abs(got - want) <= atol + rtol * np.abs(want))
