"""The Lodalix design in the engine against the plain implementation of ``plain_lodalix.py``: each
mechanism alone, whole prompts against decoding, portions down to two tokens, unequal batches, pages
and state slots that are used again, keys far back and at the edges of pages, key tiles and key
ranges, first tokens, long decoding, sizes of every kind, and greedy generation through the public
entry point."""

import json
import subprocess
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_lodalix as plain
from helpers import peak_tokens, random_tokens, replay, requests_in, trace_mixed, trace_portions, trace_tail, trace_whole

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
F = torch.float64

# worst |logit difference| of a row over the standard deviation of the request's reference logits
GATE = {"float32": 1e-4, "bfloat16": 0.1}


# ------------------------------------------------------------------ configurations
def rotary(dims, base=10000.0, scaling=None):
    rot = dict(base=base, dims=dims)
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return rot


def latent(kind=1, heads=4, dim=16, rot_dim=8, vdim=24, kv_rank=40, q_rank=24, scale=0.35, rot=None, kv_from=None):
    mixer = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, q_rank=q_rank, scale=scale,
                 rot=rot or rotary(rot_dim))
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return "latent_attention" if kind == 1 else "latent_attention_2", mixer


def delta(heads=2, dim=16, decay_rank=6):
    return "general_delta", dict(heads=heads, dim=dim, decay_rank=decay_rank)


def dense(ff=48, limit=1.0):
    return dict(kind="dense", ff=ff, limit=limit)


def config(layers, width=64, vocab=211, eps=1e-5):
    return dict(architecture="Lodalix", vocab=vocab, width=width, norm=dict(eps=eps),
                layers=[dict(type=kind, mixer=mixer, mlp=mlp) for (kind, mixer), mlp in layers])


RAMP = (4.0, 48, 6.0, 0.7)
CONFIGS = {
    # every mixer; a layer that reads an earlier layer's latent with other head counts; a layer without feed-forward
    "mixed": config([(latent(1), dense()), (delta(), dense()),
                     (latent(2, heads=3, dim=8, rot_dim=16, vdim=8, kv_rank=24, q_rank=16, rot=rotary(16, 5000.0, RAMP)), None),
                     (latent(2, heads=5, dim=8, rot_dim=16, vdim=12, kv_rank=24, q_rank=40, scale=0.2,
                             rot=rotary(16, 5000.0, RAMP), kv_from=2), dense(32, 0.4))]),
    # odd sizes: no multiple of eight anywhere, one head, a latent as large as the rotated part, part of the rotated
    # elements left unrotated, more than eight heads
    "odd": config([(latent(1, heads=1, dim=5, rot_dim=6, vdim=3, kv_rank=6, q_rank=7, scale=0.6, rot=rotary(4, 77.0)), dense(9, 3.0)),
                   (delta(heads=3, dim=7, decay_rank=1), None),
                   (latent(2, heads=11, dim=4, rot_dim=2, vdim=5, kv_rank=9, q_rank=3, rot=rotary(2, 300.0, (1.5, 8, 3.0, 0.9))), dense(5, 0.2))],
                  width=36, vocab=77, eps=1e-6),
    # sizes that reach the wide variants: heads of 64 and 128 in the recurrence, a latent above 256
    "wide": config([(delta(heads=2, dim=64, decay_rank=16), dense(64)),
                    (latent(2, heads=8, dim=32, rot_dim=32, vdim=32, kv_rank=288, q_rank=48, scale=0.15,
                            rot=rotary(32, 10000.0, (2.0, 64, 32.0, 1.0))), dense(64)),
                    (delta(heads=1, dim=128, decay_rank=8), None)], width=128, vocab=300),
    # no attention at all: no pages, only state slots
    "recurrent": config([(delta(heads=2, dim=16), dense(24)), (delta(heads=4, dim=8, decay_rank=3), None)], width=32, vocab=90),
}
PAGE = {"mixed": 4, "odd": 8, "wide": 16, "recurrent": 8}
# N(0, 0.05) weights leave scores, sinks, biases and the recurrence's rates close to nothing
SCALES = {"mix.uq": 3.0, "mix.dkv": 2.0, "mix.uk": 2.0, "mix.uv": 2.0, "mix.sink": 30.0, "mix.g": 4.0,
          "mix.k": 2.0, "mix.v": 2.0, "mix.r": 2.0, "mix.w1": 6.0, "mix.w2": 12.0, "mix.w0": 20.0, "mix.a": 4.0,
          ".b": 8.0, "mlp.gate": 3.0, "mlp.up": 3.0, "mlp.down": 3.0, "norm1": 6.0, "final.norm": 6.0,
          "embed": 20.0, "head": 6.0}
SCALES_BF16 = dict(SCALES, **{"mix.uq": 1.5, "mix.uk": 1.5})


def make_model(folder, raw, seed, std=0.05, scales=None):
    from cloud_inference_from_scratch_b200.weights import write_random_model

    return write_random_model(folder, raw, seed, std=std, scales=scales or SCALES)


class Folders:
    def __init__(self, root):
        self.sharp = {name: make_model(root / "sharp" / name, raw, 5 + index)
                      for index, (name, raw) in enumerate(CONFIGS.items())}
        self.mild = {name: make_model(root / "mild" / name, raw, 5 + index, scales=SCALES_BF16)
                     for index, (name, raw) in enumerate(CONFIGS.items())}

    def get(self, name, dtype="float32"):
        return (self.mild if dtype == "bfloat16" else self.sharp)[name]

    def __getitem__(self, name):
        return self.sharp[name]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return Folders(tmp_path_factory.mktemp("lodalix"))


def core_for(folder, dtype, page, pages, slots=4, step_tokens=0):
    from cloud_inference_from_scratch_b200.engine.core import build_core

    return build_core(folder, dtype=dtype, page_size=page, num_pages=pages, max_requests=slots,
                      max_model_len=pages * page, max_tokens_per_step=step_tokens)


def check(folder, got, dtype, gate=None):
    """Every row against the plain model run on the whole request."""
    raw, tensors = plain.read_folder(folder)
    worst = 0.0
    for rid, tokens in got["fed"].items():
        ref = plain.forward(raw, tensors, tokens).numpy()
        rows = got["logits"][rid]
        assert sorted(rows) == list(range(len(tokens))), f"{rid}: positions missing"
        mine = np.stack([rows[p] for p in range(len(tokens))])
        errors = np.abs(mine - ref).max(axis=1) / ref.std()
        if dtype == "bfloat16" and plain.first_token_delta_margin(raw, tensors, tokens) < 0.02:
            errors[0] = 0.0       # rounding decides the sign of a delta head's first output (see the oracle)
        worst = max(worst, float(errors.max()))
        limit = gate or GATE[dtype]
        assert errors.max() <= limit, (
            f"{rid}: first wrong position {int(np.argmax(errors > limit))} of {len(tokens)}, error {errors.max():.3e}")
    return worst


def run_trace(core, steps):
    return {"logits": replay(core, steps), "fed": requests_in(steps)}


def requests_for(raw, lengths, seed):
    return {f"r{i}": random_tokens(raw["vocab"], n, seed + i) for i, n in enumerate(lengths)}


# ------------------------------------------------------------------ the whole model, every cutting
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompts_decoding_portions_and_batches(folders, name, dtype):
    raw = CONFIGS[name]
    page = PAGE[name]
    # lengths: one token, two, a page's edge and one past it, a key tile's edge, several pages
    requests = requests_for(raw, [1, 2, page, page + 1, 33, 61, 97], seed=10)
    for steps in (trace_whole(requests), trace_tail(requests, tail=40), trace_portions(requests),
                  trace_mixed(requests, seed=3, live_limit=3)):
        # a pool that holds what is live and no more, and three slots: pages and slots come back
        pages = -(-peak_tokens(steps, round_to=page) // page) + 1
        core = core_for(folders.get(name, dtype), dtype, page, pages, slots=3)
        check(folders.get(name, dtype), run_trace(core, steps), dtype)
        assert core.cache.free_pages(0) == core.cache.total_pages(0)


def drawn_configuration(seed):
    """A configuration drawn from the whole space of sizes: widths, the three mixers in any order, head
    counts from one to twelve, plain, rotated and value sizes that are and are not multiples of eight,
    latents from a few elements to several hundred, rotations with and without a ramp that cover all
    or part of the rotated elements, layers that read an earlier layer's latent, heads of the
    recurrence up to 128, feed-forwards present or not with tight and loose limits."""
    import random

    rng = random.Random(seed)
    layers = []
    for index in range(rng.randint(1, 5)):
        pick = rng.random()
        owners = [i for i, layer in enumerate(layers) if layer["type"] == "latent_attention_2" and "kv_from" not in layer["mixer"]]
        if pick < 0.35:
            kind, mixer = delta(heads=rng.choice([1, 2, 3, 6]), dim=rng.choice([4, 12, 32, 33, 64, 96, 128]),
                                decay_rank=rng.choice([1, 4, 8, 24]))
        else:
            second = pick > 0.6
            rot_dim = rng.choice([2, 4, 8, 16, 24, 64])
            dims = rot_dim if rng.random() < 0.7 else max(2, rot_dim // 2 // 2 * 2)
            scaling = None
            if second and rng.random() < 0.8:
                scaling = (rng.choice([1.5, 2.0, 8.0, 40.0]), rng.choice([16, 64, 2048]), rng.choice([4.0, 32.0]), rng.choice([0.5, 1.0]))
            kind, mixer = latent(2 if second else 1, heads=rng.choice([1, 2, 4, 7, 8, 12]), dim=rng.choice([4, 8, 24, 32, 64]),
                                 rot_dim=rot_dim, vdim=rng.choice([4, 8, 20, 32, 80]), kv_rank=rng.choice([8, 24, 64, 96, 160, 320]),
                                 q_rank=rng.choice([8, 24, 40, 96]), scale=rng.choice([0.1, 0.2, 0.4]),
                                 rot=rotary(dims, rng.choice([100.0, 10000.0, 1e6]), scaling))
            if second and owners and rng.random() < 0.5:
                source = rng.choice(owners)
                shared = layers[source]["mixer"]
                mixer.update(kv_from=source, kv_rank=shared["kv_rank"], rot_dim=shared["rot_dim"], rot=shared["rot"])
        mlp = dense(rng.choice([8, 20, 64, 100]), rng.choice([0.3, 1.5, 7.0])) if rng.random() < 0.8 else None
        layers.append(dict(type=kind, mixer=mixer, mlp=mlp))
    return dict(architecture="Lodalix", vocab=rng.choice([50, 211, 448]), width=rng.choice([40, 64, 96, 128, 256]),
                norm=dict(eps=rng.choice([1e-6, 1e-5])), layers=layers)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8])
def test_drawn_configurations(seed, tmp_path):
    raw = drawn_configuration(seed)
    requests = requests_for(raw, [1, 2, 37, 150], seed=seed)
    for dtype, scales, gate in (("float32", SCALES, 4e-4), ("bfloat16", SCALES_BF16, 0.2)):
        folder = make_model(tmp_path / dtype, raw, 100 + seed, scales=scales)
        for steps in (trace_whole(requests), trace_mixed(requests, seed=seed, live_limit=3)):
            pages = -(-peak_tokens(steps, round_to=16) // 16) + 1
            core = core_for(folder, dtype, 16, pages, slots=3)
            check(folder, run_trace(core, steps), dtype, gate=gate)


def test_float32_rows_do_not_depend_on_the_cut_or_the_batch(folders):
    """The same position through four cuttings: equal to rounding of the order of additions at most."""
    raw = CONFIGS["mixed"]
    requests = requests_for(raw, [50, 31, 77], seed=40)
    seen = []
    for steps in (trace_whole(requests), trace_tail(requests, tail=20), trace_portions(requests),
                  trace_mixed(requests, seed=9, live_limit=3)):
        core = core_for(folders["mixed"], "float32", 4, 64, slots=3)
        seen.append(replay(core, steps))
    for rid, tokens in requests.items():
        base = np.stack([seen[0][rid][p] for p in range(len(tokens))])
        for other in seen[1:]:
            mine = np.stack([other[rid][p] for p in range(len(tokens))])
            assert np.abs(mine - base).max() <= 2e-5 * base.std()


def test_long_decoding_over_pages_tiles_and_key_ranges(folders):
    """300 tokens decoded one by one after a short prompt: the context grows over many pages, over the
    32-key tiles and the 128-key ranges of the attention kernel, and the recurrent state is carried
    for every token."""
    raw = CONFIGS["mixed"]
    requests = requests_for(raw, [310, 265], seed=70)
    steps = trace_tail(requests, tail=300)
    for dtype in ("float32", "bfloat16"):
        core = core_for(folders.get("mixed", dtype), dtype, 4, 150, slots=2)
        check(folders.get("mixed", dtype), run_trace(core, steps), dtype)


def test_a_state_slot_that_is_used_again_starts_from_zero(folders):
    """One slot only: every request inherits the slot of the one before it."""
    raw = CONFIGS["recurrent"]
    requests = requests_for(raw, [30, 8, 19], seed=90)
    core = core_for(folders["recurrent"], "float32", 8, 6, slots=1)
    check(folders["recurrent"], run_trace(core, trace_portions(requests)), "float32")


def test_a_model_whose_decay_width_only_the_file_knows(folders, tmp_path):
    import shutil

    folder = tmp_path / "model"
    shutil.copytree(folders["mixed"], folder)
    raw = json.loads((folder / "config.json").read_text())
    del raw["layers"][1]["mixer"]["decay_rank"]
    (folder / "config.json").write_text(json.dumps(raw))
    requests = requests_for(raw, [21], seed=3)
    core = core_for(folder, "float32", 4, 8, slots=1)
    check(folder, run_trace(core, trace_whole(requests)), "float32")


# ------------------------------------------------------------------ mechanisms alone
def runtime(dtype):
    from cloud_inference_from_scratch_b200.engine.runtime import Runtime

    return Runtime("cuda:0", dtype)


def rand(*shape, scale=1.0, seed=0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


def close(got, want, dtype, scale=None, loose=3e-2):
    want = want.double().cpu()
    error = float((got.double().cpu() - want).abs().max() / (scale or want.std()))
    assert error <= (2e-5 if dtype == "float32" else loose), error


def fake_step(lengths, contexts, page, dtype, rank, rot, seed=0):
    """Positions, tables and empty pools for requests that hold ``contexts`` tokens and bring ``lengths``;
    pages are dealt out in a shuffled order."""
    total = [c + n for c, n in zip(contexts, lengths)]
    pages_per = [-(-t // page) for t in total]
    order = torch.randperm(sum(pages_per) + 2, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.full((len(lengths), max(pages_per)), -1, dtype=torch.int32)
    cursor = 0
    for r, count in enumerate(pages_per):
        table[r, :count] = torch.tensor(order[cursor:cursor + count], dtype=torch.int32)
        cursor += count
    positions = torch.cat([torch.arange(c, c + n) for c, n in zip(contexts, lengths)]).int()
    request_of = torch.cat([torch.full((n,), r) for r, n in enumerate(lengths)]).int()
    kv = SimpleNamespace(group=0, num_pages=len(order), page_size=page,
                         k=torch.zeros(len(order), 1, page, rank, dtype=dtype).cuda(),
                         v=torch.zeros(len(order), 1, page, rot, dtype=dtype).cuda())
    ctx = SimpleNamespace(positions=positions.cuda(), request_of_token=request_of.cuda(), block_tables=[table.cuda()],
                          num_requests=len(lengths))
    return ctx, kv, table


def rotation_of(rot, pairing, device="cuda"):
    f, magnitude = plain.rotary_frequencies(rot)
    return SimpleNamespace(inv_freq=f.float().to(device), magnitude=magnitude, interleaved=pairing == "interleaved",
                           dims=rot["dims"])


def rows_in_pages(pool, table, request, count, page):
    return torch.stack([pool[int(table[request, p // page]), 0, p % page] for p in range(count)]).double().cpu()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("pairing", ["interleaved", "half"])
@pytest.mark.parametrize("q_rank,rank,rot_dim,dims", [(24, 40, 8, 8), (7, 6, 6, 4), (96, 512, 64, 64), (3, 9, 2, 2)])
def test_latent_rows_are_normalised_rotated_and_paged(dtype, pairing, q_rank, rank, rot_dim, dims):
    """The kernel behind the down projection against the oracle's ``latent_keys``: both norms, both
    pairings, a rotation that covers part of the rotated elements, positions that start in mid-page."""
    rt = runtime(dtype)
    rot = rotary(dims, 3000.0, (3.0, 40, 5.0, 0.8) if pairing == "half" else None)
    page, eps = 8, 1e-5
    lengths, contexts = [1, 13, 30], [21, 0, 5]
    tokens = sum(lengths)
    ctx, kv, table = fake_step(lengths, contexts, page, rt.dtype, rank, rot_dim)
    down = rand(tokens, q_rank + rank + rot_dim, seed=1, scale=2.0)
    q_gain, kv_gain = 1 + rand(q_rank, scale=0.3, seed=2), 1 + rand(rank, scale=0.3, seed=3)
    q_out = torch.empty(tokens, q_rank, dtype=rt.dtype).cuda()
    rt.ops.latent_prepare(down.cuda(), q_out, q_gain.cuda(), kv_gain.cuda(), ctx, kv, rotation_of(rot, pairing), q_rank,
                          rank, rot_dim, eps, True, True)
    rt.ops.check_errors()
    close(q_out, plain.plain_gain_norm(down[:, :q_rank].double(), q_gain.double(), eps), dtype)
    # the oracle takes the projection apart itself: give it an identity down projection
    p = {"mix.dkv": torch.eye(rank + rot_dim, dtype=F), "mix.dkv.norm": kv_gain.double()}
    first = 0
    for r, (n, c) in enumerate(zip(lengths, contexts)):
        want_latent, want_key = plain.latent_keys(down[first:first + n, q_rank:].double(), p, dict(kv_rank=rank, rot=rot), eps, c, pairing)
        got_latent = rows_in_pages(kv.k, table, r, c + n, page)[c:]
        got_key = rows_in_pages(kv.v, table, r, c + n, page)[c:]
        close(got_latent, want_latent, dtype, scale=1.0)
        close(got_key, want_key, dtype, scale=float(want_key.abs().max()))
        first += n
    # a layer that only reads writes nothing
    before = kv.k.clone()
    rt.ops.latent_prepare(down.cuda() * 2, q_out, q_gain.cuda(), None, ctx, kv, rotation_of(rot, pairing), q_rank, rank,
                          rot_dim, eps, False, False)
    assert torch.equal(before, kv.k)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("heads,depth,width,tokens", [(3, 16, 40, 5), (1, 5, 3, 33), (9, 130, 129, 17), (2, 64, 512, 1)])
def test_products_per_head(dtype, heads, depth, width, tokens):
    rt = runtime(dtype)
    x = rand(tokens, heads * (depth + 3), seed=1)
    w = rand(heads, depth, width, seed=2, scale=0.3).to(rt.dtype)
    gate = rand(tokens, heads * width + 2, seed=3)
    want = torch.einsum("thk,hkn->thn", x.view(tokens, heads, depth + 3)[..., :depth].double(), w.double())
    out = torch.empty(tokens, heads * width, dtype=torch.float32).cuda()
    rt.ops.head_linear(x.cuda(), depth + 3, w.cuda(), out, width, heads)
    # more than 16 tokens in bfloat16 go through a batched library product with a bfloat16 result
    close(out.view(tokens, heads, width), want, "float32" if tokens <= 16 else dtype)
    gated = torch.empty(tokens, heads * width, dtype=rt.dtype).cuda()
    rt.ops.head_linear(x.cuda(), depth + 3, w.cuda(), gated, width, heads, gate=gate.cuda()[:, 2:])
    close(gated.view(tokens, heads, width), want * torch.sigmoid(gate[:, 2:].double()).view(tokens, heads, width), dtype)


def attention_oracle(q_latent, q_rot, latent_rows, key_rows, position, scale, sink):
    """Weighted sum of latents for one query: q_latent [heads, rank], q_rot [heads, rot] (already rotated)."""
    seen = position + 1
    score = (q_latent.double() @ latent_rows[:seen].double().T + q_rot.double() @ key_rows[:seen].double().T) * scale
    top = score.max(dim=1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.double().view(-1, 1))
    weight = torch.exp(score - top)
    total = weight.sum(dim=1, keepdim=True)
    if sink is not None:
        total = total + torch.exp(sink.double().view(-1, 1) - top)
    return (weight / total) @ latent_rows[:seen].double()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("with_sink", [False, True])
@pytest.mark.parametrize("context", [0, 15, 16, 31, 32, 33, 127, 128, 129, 700])
def test_attention_over_latent_rows_with_one_key_that_stands_out(dtype, with_sink, context):
    """A single query (keys cut into ranges over CTAs) and the same query as the last row of a portion
    (one CTA walks all keys): the first key, the key at the last place of a page, a 32-key tile or a
    128-key range, or one far back among hundreds is made to carry nearly all the weight of one head,
    and the newest key that of another; a sink so large that it halves one head's output."""
    rt = runtime(dtype)
    heads, rank, rot_dim, page, scale = 3, 24, 8, 16, 0.5
    rot = rotary(rot_dim, 100.0)
    n = context + 1
    latent_rows = rand(n, rank, seed=1).to(rt.dtype)
    key_rows = rand(n, rot_dim, seed=2).to(rt.dtype)
    q_latent, q_raw = rand(n, heads * rank, seed=3), rand(n, heads * (rot_dim + 5), seed=4)
    stand_out = {0: 0, 15: 15, 16: 15, 31: 31, 32: 31, 33: 32, 127: 127, 128: 127, 129: 128, 700: 2}[context]
    q_latent[n - 1, :rank] = latent_rows[stand_out].float() * (20.0 / float(latent_rows[stand_out].float().norm()) ** 2 / scale)
    q_latent[n - 1, rank:2 * rank] = latent_rows[n - 1].float() * (20.0 / float(latent_rows[n - 1].float().norm()) ** 2 / scale)
    sink = torch.tensor([-30.0, 0.5, 4.0]) if with_sink else None
    if with_sink:      # head 0's sink equals its largest score: half of the weight goes nowhere
        rotated = plain.rotate(q_raw.view(n, heads, rot_dim + 5)[n - 1:, :, 5:].double(), torch.tensor([n - 1]), rot, "interleaved")[0]
        score = (q_latent[n - 1, :rank].double() @ latent_rows.double().T + rotated[0] @ key_rows.double().T) * scale
        sink[0] = float(score.max())
    for lengths, contexts in (([1], [context]), ([n], [0])):
        ctx, kv, table = fake_step(lengths, contexts, page, rt.dtype, rank, rot_dim, seed=context)
        for p in range(n):
            kv.k[int(table[0, p // page]), 0, p % page] = latent_rows[p].cuda()
            kv.v[int(table[0, p // page]), 0, p % page] = key_rows[p].cuda()
        rows = slice(n - lengths[0], n)
        out = torch.zeros(lengths[0], heads * rank, dtype=torch.float32).cuda()
        rt.ops.latent_attention(q_latent[rows].contiguous().cuda(), q_raw[rows].contiguous().cuda()[:, 5:], rot_dim + 5, out, ctx, kv,
                                rotation_of(rot, "interleaved"), sink.cuda() if with_sink else None, heads, rank, rot_dim, scale)
        rt.ops.check_errors()
        for row, position in enumerate(range(n - lengths[0], n)):
            rotated = plain.rotate(q_raw.view(n, heads, rot_dim + 5)[position:position + 1, :, 5:].double(),
                                   torch.tensor([position]), rot, "interleaved")[0]
            want = attention_oracle(q_latent[position].view(heads, rank), rotated, latent_rows, key_rows, position, scale, sink)
            close(out[row].view(heads, rank), want, dtype, scale=1.0, loose=4e-2)
        last = out[-1].view(heads, rank).double().cpu()
        share = 0.5 if with_sink else 1.0
        assert (last[0] - share * latent_rows[stand_out].double()).abs().max() < 0.05
        if 0 < context < 700:      # among 700 random keys the newest one's lead is not safe
            assert (last[1] - latent_rows[n - 1].double()).abs().max() < 0.05 + (0.2 if with_sink else 0.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rank,rot_dim,heads", [(512, 64, 16), (640, 16, 3), (1024, 8, 2), (72, 24, 20)])
def test_attention_over_wide_latents_and_many_heads(dtype, rank, rot_dim, heads):
    """Latents at and above what the tensor-core kernel takes, more heads than one tile of 16 rows, a
    portion whose tokens pair up in CTAs next to single queries of other requests."""
    rt = runtime(dtype)
    page, scale = 16, 1.5 / rank ** 0.5
    rot = rotary(rot_dim, 1000.0)
    lengths, contexts = [1, 1, 71, 2], [130, 0, 0, 64]
    tokens = sum(lengths)
    ctx, kv, table = fake_step(lengths, contexts, page, rt.dtype, rank, rot_dim, seed=3)
    rows = [(rand(c + n, rank, seed=10 + r).to(rt.dtype), rand(c + n, rot_dim, seed=20 + r).to(rt.dtype))
            for r, (n, c) in enumerate(zip(lengths, contexts))]
    for r, (latent_rows, key_rows) in enumerate(rows):
        for p in range(latent_rows.shape[0]):
            kv.k[int(table[r, p // page]), 0, p % page] = latent_rows[p].cuda()
            kv.v[int(table[r, p // page]), 0, p % page] = key_rows[p].cuda()
    q_latent, q_raw = rand(tokens, heads * rank, seed=5), rand(tokens, heads * rot_dim, seed=6)
    sink = rand(heads, seed=7)
    out = torch.zeros(tokens, heads * rank, dtype=torch.float32).cuda()
    rt.ops.latent_attention(q_latent.cuda(), q_raw.cuda(), rot_dim, out, ctx, kv, rotation_of(rot, "interleaved"), sink.cuda(),
                            heads, rank, rot_dim, scale)
    rt.ops.check_errors()
    row = 0
    for r, (n, c) in enumerate(zip(lengths, contexts)):
        for position in range(c, c + n):
            rotated = plain.rotate(q_raw[row].view(1, heads, rot_dim).double(), torch.tensor([position]), rot, "interleaved")[0]
            want = attention_oracle(q_latent[row].view(heads, rank), rotated, rows[r][0], rows[r][1], position, scale, sink)
            close(out[row].view(heads, rank), want, dtype, scale=1.0, loose=4e-2)
            row += 1


@pytest.mark.parametrize("first_lengths", [[13, 1, 6], [40, 3, 33]])      # the second: the two-kernel form for portions
@pytest.mark.parametrize("dim", [1, 7, 16, 33, 64, 100, 128, 160, 256])
def test_delta_scan_carries_its_state_between_steps_and_leaves_padding_rows_alone(dim, first_lengths):
    rt = runtime("float32")
    heads = 3
    lengths = list(first_lengths)
    width = heads * dim
    slots = torch.tensor([2, 0, 3], dtype=torch.int32)
    state = torch.zeros(5, heads, dim, dim).cuda()
    w0, a0 = rand(width, seed=1), rand(width, seed=2)
    history = {r: [] for r in range(3)}
    for step, active in enumerate(([1, 1, 1], [1, 0, 1], [1, 1, 1])):
        tokens = sum(lengths)
        proj = rand(tokens, 5 * width + 2, seed=20 + step)
        decay = rand(tokens, width, seed=40 + step, scale=2.0)
        starts = torch.tensor([0, *np.cumsum(lengths)], dtype=torch.int32)
        ctx = SimpleNamespace(query_start=starts.cuda(), slots=slots.cuda(), num_requests=3,
                              request_active=torch.tensor(active, dtype=torch.int32).cuda())
        out = torch.empty(tokens, width, dtype=torch.float32).cuda()
        # r, k, v and the removal projection in another order than the mixer keeps them
        rt.ops.delta_scan(proj.cuda(), (2 * width, 0, 4 * width + 2, width), decay.cuda(), w0.cuda(), a0.cuda(), out, state, ctx,
                          heads, dim)
        rt.ops.check_errors()
        for r in range(3):
            rows = proj[starts[r]:starts[r + 1]].double()
            shape = (-1, heads, dim)
            k, a, rr, v = (rows[:, o:o + width].view(shape) for o in (0, width, 2 * width, 4 * width + 2))
            w = torch.exp(-np.exp(-0.5) * torch.sigmoid(decay[starts[r]:starts[r + 1]].double() + w0.double())).view(shape)
            before = history[r][-1] if history[r] else None
            want, after = plain.delta_recurrence(rr, k, v, w, torch.sigmoid(a.reshape(-1, width) + a0.double()).view(shape), before)
            close(out[starts[r]:starts[r + 1]].view(shape), want, "float32", scale=max(1.0, float(want.abs().max())))
            if active[r]:
                history[r].append(after)
            held = history[r][-1] if history[r] else torch.zeros(heads, dim, dim)
            close(state[slots[r]], held, "float32", scale=max(1.0, float(after.abs().max())))
        lengths = [1, 1, 4]
    assert float(state[1].abs().max()) == 0 and float(state[4].abs().max()) == 0      # other slots untouched


@pytest.mark.parametrize("dim", [12, 64, 128])
def test_delta_rule_in_one_kernel_and_in_two_kernels_agree(monkeypatch, dim):
    rt = runtime("float32")
    heads, lengths = 2, [50, 9, 31]
    width, tokens = heads * dim, sum(lengths)
    proj, decay = rand(tokens, 5 * width, seed=1), rand(tokens, width, seed=2)
    w0, a0 = rand(width, seed=3), rand(width, seed=4)
    starts = torch.tensor([0, *np.cumsum(lengths)], dtype=torch.int32)
    ctx = SimpleNamespace(query_start=starts.cuda(), slots=torch.tensor([1, 0, 2], dtype=torch.int32).cuda(), num_requests=3,
                          request_active=torch.ones(3, dtype=torch.int32).cuda())
    seen = []
    for switch in ("1", "0"):
        monkeypatch.setenv("CIE_DELTA_STREAM", switch)
        state = rand(3, heads, dim, dim, seed=5, scale=0.3).cuda()
        out = torch.empty(tokens, width, dtype=torch.float32).cuda()
        rt.ops.delta_scan(proj.cuda(), (0, width, 2 * width, 4 * width), decay.cuda(), w0.cuda(), a0.cuda(), out, state, ctx, heads, dim)
        rt.ops.check_errors()
        seen.append((out.cpu(), state.cpu()))
    close(seen[0][0], seen[1][0], "float32", scale=float(seen[1][0].abs().max()))
    close(seen[0][1], seen[1][1], "float32", scale=float(seen[1][1].abs().max()))


def test_delta_rule_unlearns_along_its_key():
    """With removal rate 1 and no decay, writing a key a second time REPLACES what it held: the
    first value is gone and the read gives the second."""
    heads, dim = 1, 8
    k = torch.zeros(2, heads, dim, dtype=F)
    k[:, 0, 3] = 1.0
    v = rand(2, heads, dim, seed=1).double()
    ones = torch.ones(2, heads, dim, dtype=F)
    out, _ = plain.delta_recurrence(k, k, v, ones, ones)
    assert torch.allclose(out[1, 0], v[1, 0], atol=1e-5)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_norm_with_gate_and_clamped_activation(dtype):
    rt = runtime(dtype)
    tokens, groups, size = 7, 3, 20
    o = rand(tokens, groups * size, seed=1, scale=3.0)
    gate = rand(tokens, groups * size + 4, seed=2)
    gain = 1 + rand(groups * size, seed=3, scale=0.3)
    out = torch.empty(tokens, groups * size, dtype=rt.dtype).cuda()
    rt.ops.group_gate_norm(o.cuda(), gate.cuda()[:, 4:], gain.cuda(), 1e-3, out, groups)
    want = plain.rms_divide(o.double().view(tokens, groups, size), 1e-3).reshape(tokens, -1) * gain.double() * torch.sigmoid(gate[:, 4:].double())
    close(out, want, dtype)
    # the activation: gates above the limit are capped, ups beyond it on either side are clamped
    inter, limit = 33, 0.7
    both = rand(tokens, 2 * inter, seed=4, scale=1.5)
    bias = rand(2 * inter, seed=5, scale=0.5)
    hidden = torch.empty(tokens, inter, dtype=rt.dtype).cuda()
    rt.ops.gated_act(both.cuda(), bias.cuda(), hidden, 1.702, limit, 1.0)
    full = both.double() + bias.double()
    g, u = full[:, :inter].clamp(max=limit), full[:, inter:].clamp(-limit, limit)
    assert (full[:, :inter] > limit).any() and (full[:, inter:] < -limit).any() and (full[:, :inter] < -limit).any()
    close(hidden, g * torch.sigmoid(1.702 * g) * (u + 1.0), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_parts_alone_against_the_plain_sublayers(dtype):
    """The feed-forward and the delta mixer as parts, with their own tensor names."""
    from cloud_inference_from_scratch_b200.config import PartSpec
    from cloud_inference_from_scratch_b200.parts import build_part

    rt = runtime(dtype)
    hidden, ff, tokens = 40, 24, 19
    part = build_part("feed_forward", PartSpec("clamped_glu", dict(hidden_size=hidden, intermediate_size=ff, limit=0.5)))
    tensors = {"gate": rand(ff, hidden, scale=0.3, seed=1).to(rt.dtype), "up": rand(ff, hidden, scale=0.3, seed=2).to(rt.dtype),
               "down": rand(hidden, ff, scale=0.3, seed=3).to(rt.dtype), "gate.b": rand(ff, seed=4, scale=0.3),
               "up.b": rand(ff, seed=5, scale=0.3), "down.b": rand(hidden, seed=6)}
    assert set(part.tensor_specs()) == set(tensors)
    part.bind({name: value.cuda() for name, value in tensors.items()}, rt)
    x = rand(tokens, hidden, seed=7).to(rt.dtype)
    got = part.forward(x.cuda(), None)
    assert got.dtype == torch.float32
    close(got, plain.clamped_glu(x.double(), {"mlp." + name: value.double() for name, value in tensors.items()}, 0.5), dtype)
    # the norm whose stored weight is an offset from one
    norm = build_part("norm", PartSpec("rmsnorm", dict(hidden_size=hidden, eps=1e-5, gain_offset=1.0, name="")))
    weight = rand(hidden, seed=8, scale=0.4)
    norm.bind({"": weight.cuda()}, rt)
    residual = rand(tokens, hidden, seed=9, scale=3.0).cuda()
    close(norm.forward(residual, None, None), plain.offset_gain_norm(residual.double().cpu(), weight.double(), 1e-5), dtype)


# ------------------------------------------------------------------ the public entry point
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk,active", [(8, 3), (24, 1)])
def test_greedy_generation_through_the_engine(folders, dtype, chunk, active):
    """Through the scheduler, the runner's captured decode steps and the sampler.  The second setting runs the
    requests one after the other with portions of 24 tokens: the long prompts come when decode steps have
    been captured already, so whatever their kernels keep by the token must have its full size by then."""
    from cloud_inference_from_scratch_b200 import generate

    raw, tensors = plain.read_folder(folders.get("mixed", dtype))
    prompts = [random_tokens(raw["vocab"], n, 100 + n) for n in (1, 9, 30, 17)]
    results = generate(folders.get("mixed", dtype), prompts, max_output_tokens=12, dtype=dtype, block_size=4,
                       kv_cache_blocks=40, prefill_chunk_size=chunk, max_batched_tokens=chunk + 12,
                       max_active_sequences=active)
    for prompt, result in zip(prompts, results):
        got = result.token_ids
        assert len(got) == 12
        # every token is the argmax of the plain model's logits given the engine's own tokens so far
        # (a near tie may go the other way under bfloat16 rounding: then the logits must be close)
        logits = plain.forward(raw, tensors, prompt + got).numpy()
        for index, token in enumerate(got):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - (1e-3 if dtype == "float32" else 0.15) * logits.std()


def test_trace_program_replays_a_lodalix_model(folders, tmp_path):
    raw, tensors = plain.read_folder(folders["odd"])
    tokens = random_tokens(raw["vocab"], 21, 7)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": tokens[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": tokens[13:], "want": [7]},
                                     {"id": "b", "tokens": tokens[:2], "want": []}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    done = subprocess.run([str(ROOT / "bin" / "trace_run"), "--model", str(folders["odd"]), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [line for line in done.stdout.splitlines() if line.startswith("done")] == ["done 0", "done 1"]
    ref = plain.forward(raw, tensors, tokens).numpy()
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    second = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    assert np.abs(first - ref[[0, 12]]).max() <= 1e-4 * ref.std()
    assert np.abs(second - ref[[20]]).max() <= 1e-4 * ref.std()
