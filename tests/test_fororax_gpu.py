"""The Fororax design through the engine against the plain implementation (``tests/plain/fororax_plain.py``): every
mixer alone and together, whole prompts, decoding through the pages, portions down to two tokens, mixed batches with
pages that are used again, other sizes, both precisions, greedy generation through ``LLMEngine``; and the kernels of
its mechanisms alone."""
import json
import random
import tempfile
from pathlib import Path

import pytest
import torch

import helpers
from plain import fororax_plain as plain

pytestmark = pytest.mark.gpu


def moe(experts=5, identity=2, top=3, ff=40, limit=0.8, shared=(56, 1.5)):
    out = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top},
           "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def attention(heads=6, kv_heads=2, dim=24, vdim=40, kv_from=None, mlp="default", second=False, scale=None):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale or 2.0 / dim ** 0.5}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention_2" if second else "attention", "mixer": mixer, "mlp": moe() if mlp == "default" else mlp}


def attention2(**kw):
    return attention(second=True, **kw)


def model(layers, width=72, vocab=211, positions=700, alpha=2.0, embed_scale=0.5, cap=4.0, eps=1e-5):
    return {"architecture": "Fororax", "vocab": vocab, "width": width, "max_positions": positions, "layers": layers,
            "norm": {"eps": eps}, "postln_alpha": alpha, "embedding": {"scale": embed_scale}, "logit_softcap": cap}


CONFIGS = {
    "penalty_only": model([attention(), attention(kv_from=0, heads=4, mlp=moe(experts=3, identity=0, top=1, shared=None))]),
    "sink_only": model([attention2(), attention2(heads=3, kv_heads=3, dim=16, vdim=16, mlp=None)]),
    "both_kinds": model([attention2(heads=4, kv_heads=2, dim=32, vdim=32), attention(heads=4, dim=16, vdim=24),
                         attention(heads=8, dim=16, vdim=24, kv_from=1), attention2(heads=6, kv_heads=3, dim=16, vdim=8),
                         attention(heads=2, kv_heads=1, dim=64, vdim=32, mlp=moe(experts=2, identity=3, top=2))], width=80),
    # values that many models make equal or one: one key/value head, one query head per group, one expert chosen, no
    # identity experts, no shared expert, alpha and the embedding's constant one, dim = vdim
    "equal_or_one": model([attention2(heads=1, kv_heads=1, dim=32, vdim=32, mlp=moe(experts=4, identity=0, top=1, shared=None)),
                           attention(heads=3, kv_heads=3, dim=16, vdim=16, mlp=moe(experts=1, identity=1, top=2, ff=64)),
                           attention(heads=3, kv_heads=3, dim=16, vdim=16, kv_from=1, mlp=None)],
                          width=64, alpha=1.0, embed_scale=1.0, cap=30.0),
    # sizes that no vector load or few-rows product takes; more than eight query heads on one key/value head; a reader
    # of a layer that is not the first; a layer without a feed-forward in the middle
    "odd_sizes": model([attention(heads=3, kv_heads=1, dim=20, vdim=12, mlp=None),
                        attention2(heads=18, kv_heads=2, dim=10, vdim=6, mlp=moe(experts=7, identity=1, top=4, ff=18, shared=(10, 0.5))),
                        attention(heads=9, kv_heads=1, dim=12, vdim=28, mlp=moe(experts=3, identity=5, top=3, ff=50, limit=0.3)),
                        attention(heads=5, kv_heads=1, dim=12, vdim=28, kv_from=2, mlp=None),
                        attention2(heads=2, kv_heads=2, dim=36, vdim=20),
                        # a reader of the pages of a layer with biases, sink and mixing (their keys carry the bias)
                        attention(heads=4, kv_heads=2, dim=10, vdim=6, kv_from=1, mlp=None)], width=102, vocab=333, positions=900),
}
RMS_LIMIT = {"float32": 2.0e-5, "bfloat16": 1.0e-1}
_MODELS: dict = {}


def folder_of(name: str):
    if name not in _MODELS:
        holder = tempfile.TemporaryDirectory(prefix=f"fororax_{name}_")
        plain.write_model(holder.name, CONFIGS[name], seed=23 + len(_MODELS))
        _MODELS[name] = (holder, Path(holder.name), plain.load_folder(holder.name))
    return _MODELS[name][1]


def reference(name: str, tokens):
    folder_of(name)
    config, weights = _MODELS[name][2]
    return plain.forward_full(config, weights, tokens).to(torch.float32)


def replay(name: str, dtype: str, steps, max_tokens: int, page: int = 16, max_requests: int = 4):
    from llm_serving_engine_b200.engine.trace_replay import replay as run

    with tempfile.TemporaryDirectory(prefix="fororax_out_") as out:
        run(folder_of(name), dtype, out, max_tokens, [json.dumps(step) for step in steps], block_size=page,
            max_requests=max_requests)
        return helpers.collect(steps, Path(out))


def compare(name, dtype, requests, got, what):
    """Row error over logit size, per position.  float32: every row within the limit.  bfloat16: a router's choice
    between two almost equal scores may fall the other way than in the plain implementation, which moves that row by
    more than rounding does: up to one row in thirty may pass the limit, none by more than four times."""
    over = rows = 0
    for rid, tokens in requests.items():
        want = reference(name, tokens)
        assert got[rid].shape == want.shape, f"{what}: {rid}: shape {tuple(got[rid].shape)} against {tuple(want.shape)}"
        centred = want - want.mean(-1, keepdim=True)
        per_row = (got[rid] - want).double().pow(2).mean(-1).sqrt() / centred.double().pow(2).mean().sqrt()
        worst = float(per_row.max())
        hard = RMS_LIMIT[dtype] * (4.0 if dtype == "bfloat16" else 1.0)
        assert worst <= hard, (f"{what}: {name} {dtype} request {rid}: row error / logit size {worst:.2e} at position "
                               f"{int(per_row.argmax())}, first above the limit {int((per_row > hard).nonzero()[0])}")
        over += int((per_row > RMS_LIMIT[dtype]).sum())
        rows += per_row.shape[0]
    assert over <= rows // 30, f"{what}: {name} {dtype}: {over} of {rows} rows above {RMS_LIMIT[dtype]:.0e}"


def some_requests(name, lengths, seed=5):
    rng = random.Random(seed)
    vocab = CONFIGS[name]["vocab"]
    return {f"r{index}": helpers.random_tokens(rng, vocab, length) for index, length in enumerate(lengths)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(name, dtype):
    requests = some_requests(name, [1, 2, 17, 70])
    got = replay(name, dtype, helpers.trace_whole(requests), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "whole")


@pytest.mark.parametrize("name", ["both_kinds", "odd_sizes"])
def test_every_layer_against_the_plain_layers(name):
    """The float32 residual after every layer, through the engine's own step function."""
    from llm_serving_engine_b200.cache.manager import CacheManager
    from llm_serving_engine_b200.config import CacheConfig
    from llm_serving_engine_b200.engine.step import StepEntry, StepRunner
    from llm_serving_engine_b200.models import cache_requirements, load_model

    tokens = some_requests(name, [45], seed=2)["r0"]
    engine_model = load_model(folder_of(name), dtype="float32")
    cache = CacheManager(cache_requirements(engine_model.spec), CacheConfig(block_size=8, num_blocks=16), engine_model.dtype,
                         engine_model.device, engine_model.spec.max_position_embeddings, num_state_slots=2)
    runner = StepRunner(engine_model, cache, 64, 2, use_graphs=False)
    seen = []
    engine_model.layer_hook = lambda position, stream: seen.append(stream.residual.clone().cpu())
    cache.create("a")
    runner.run([StepEntry("a", tokens, [])])
    config, weights = _MODELS[name][2]
    want = plain.forward_layers(config, weights, tokens)[1:]
    assert len(seen) == len(want)
    for index, (got, expected) in enumerate(zip(seen, want)):
        assert float((got - expected).abs().max()) <= 5e-5 * float(expected.abs().max()), f"layer {index}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    """Decoding reads the pages that the prompt step left (single tokens are replayed from a captured graph)."""
    requests = some_requests(name, [40, 9, 3], seed=6)
    got = replay(name, dtype, helpers.trace_tail_decode(requests, tail=24), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "tail decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["both_kinds", "odd_sizes"])
def test_portions_of_changing_size(name, dtype):
    requests = some_requests(name, [150, 33], seed=7)
    for sizes in ((7, 2, 13, 3, 2, 31, 5, 16, 2, 64, 17), (2,), (16, 16, 1, 15, 17)):
        got = replay(name, dtype, helpers.trace_portions(requests, sizes), helpers.max_tokens_for(requests))
        compare(name, dtype, requests, got, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 8])
def test_mixed_batches_reuse_pages(dtype, page):
    """Nine requests through four slots and a pool sized for the live ones only: a page's old rows must not be read,
    and the layer that reads another layer's pages must follow that layer's tables."""
    requests = some_requests("both_kinds", [61, 5, 90, 33, 2, 47, 130, 18, 64], seed=8)
    steps, peak = helpers.trace_mixed(requests, seed=3, max_live=4)
    got = replay("both_kinds", dtype, steps, peak, page=page)
    compare("both_kinds", dtype, requests, got, "mixed")


def test_a_batch_gives_what_each_request_gives_alone():
    for name in ("both_kinds", "odd_sizes"):
        requests = some_requests(name, [37, 12, 80, 5], seed=9)
        steps, peak = helpers.trace_mixed(requests, seed=4, max_live=4)
        together = replay(name, "float32", steps, peak)
        for rid, tokens in requests.items():
            alone = replay(name, "float32", helpers.trace_whole({rid: tokens}), helpers.max_tokens_for({rid: tokens}))
            assert float((together[rid] - alone[rid]).abs().max()) <= 2e-5 * float(alone[rid].abs().max())


def test_long_decoding_crosses_key_chunks_and_many_pages():
    """600 single tokens after a short prompt: the keys pass the borders of tiles (32), chunks (256) and many pages."""
    requests = some_requests("both_kinds", [610], seed=10)
    got = replay("both_kinds", "float32", helpers.trace_tail_decode(requests, tail=600), 640)
    compare("both_kinds", "float32", requests, got, "long decoding")


def test_greedy_generation_through_the_engine_and_its_scheduler():
    """More requests than the scheduler keeps live, prompts cut into portions: every request's greedy tokens equal
    the plain implementation's (float32; a request whose top two logits are closer than the arithmetic's noise is
    skipped from that token on)."""
    from llm_serving_engine_b200.config import CacheConfig, SchedulerConfig
    from llm_serving_engine_b200.engine.llm_engine import LLMEngine
    from llm_serving_engine_b200.models import load_model
    from llm_serving_engine_b200.sampling.sampler import GenerationConfig

    name = "both_kinds"
    engine = LLMEngine(load_model(folder_of(name), dtype="float32"), None,
                       cache_config=CacheConfig(block_size=16, num_blocks=40),
                       scheduler_config=SchedulerConfig(max_batch_size=3, max_tokens_per_step=48), prefill_chunk_size=20)
    prompts = list(some_requests(name, [30, 7, 55, 2, 19, 41], seed=12).values())
    new_tokens = 12
    produced = engine.generate_many(prompts, GenerationConfig(max_new_tokens=new_tokens, temperature=0.0))
    for prompt, tokens in zip(prompts, produced):
        assert len(tokens) == new_tokens
        logits = reference(name, prompt + tokens)
        for index, token in enumerate(tokens):
            row = logits[len(prompt) + index - 1]
            top = torch.topk(row, 2).values
            if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
                break
            assert int(row.argmax()) == token, f"token {index} of a {len(prompt)}-token prompt"


# ------------------------------------------------------------------ the mechanisms' kernels alone
def _paged(keys, values, page, spare=5, seed=0):
    """Scatter keys [T, G, dk] and values [T, G, dv] of one request over the pages of a larger pool whose other rows
    hold NaN.  Returns (k_cache, v_cache, block table [1, pages])."""
    count, groups = keys.shape[0], keys.shape[1]
    pages = -(-count // page)
    order = torch.randperm(pages + spare, generator=torch.Generator().manual_seed(seed))[:pages].to(torch.int32)
    k_cache = torch.full((pages + spare, groups, page, keys.shape[2]), float("nan"))
    v_cache = torch.full((pages + spare, groups, page, values.shape[2]), float("nan"))
    for logical in range(pages):
        rows = slice(logical * page, min(count, (logical + 1) * page))
        size = rows.stop - rows.start
        k_cache[int(order[logical]), :, :size] = keys[rows].transpose(0, 1)
        v_cache[int(order[logical]), :, :size] = values[rows].transpose(0, 1)
        k_cache[int(order[logical]), :, size:] = 0.0
        v_cache[int(order[logical]), :, size:] = 0.0
    return k_cache, v_cache, order.view(1, -1)


def _plain_rows(q, keys, values, positions, scale, r1=None, r2=None, sink=None, table=None):
    """Rows of the plain attention: q [R, H, dk] at ``positions`` over keys/values [T, G, *]."""
    count = keys.shape[0]
    full_q = torch.zeros(count, q.shape[1], q.shape[2], dtype=torch.float64)
    scores = []
    for row, pos in enumerate(positions):
        full_q[pos] = q[row].double()
    scores = plain.causal_scores(full_q, keys.double(), scale)
    if r1 is not None:
        scores = scores - plain.distance_penalty(count, r1.double(), r2.double())
    weights = plain.softmax_with_sink(scores, None if sink is None else sink.double())
    if table is not None:
        weights = plain.mix_heads(weights, table.double())
    out = plain.apply_weights(weights, values.double())
    return out[torch.tensor(positions)].view(len(positions), q.shape[1], -1)


def _attend(q, k_cache, v_cache, table, positions, scale, dtype, r1=None, r2=None, sink=None, mix=None, split=None):
    from llm_serving_engine_b200.kernels import ops

    count, heads, groups, dv = q.shape[0], q.shape[1], k_cache.shape[1], v_cache.shape[3]
    device = lambda t: None if t is None else t.cuda()
    seg = torch.zeros(count, dtype=torch.int32, device="cuda")
    pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
    common = (table.cuda(), seg, pos, scale, device(r1), device(r2), device(sink))
    if mix is None:
        out = torch.empty(count, heads, dv, dtype=dtype, device="cuda")
        ops.attention_scored(q.to(dtype).cuda(), k_cache.to(dtype).cuda(), v_cache.to(dtype).cuda(), out, *common, split=split)
        return out.float().cpu()
    cross = groups > 1
    wide = torch.empty(count, heads, groups if cross else 1, dv, dtype=torch.float32, device="cuda")
    ops.attention_scored(q.to(dtype).cuda(), k_cache.to(dtype).cuda(), v_cache.to(dtype).cuda(), wide, *common, cross=cross, split=split)
    out = torch.empty(count, heads * dv, dtype=dtype, device="cuda")
    ops.head_mix_gate(wide, mix.cuda(), None, 0, None, seg, out, heads, groups, dv)
    return out.float().cpu().view(count, heads, dv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["penalty", "sink_mixed"])
def test_attention_finds_one_far_key_at_every_border(dtype, kind):
    """One key among hundreds is made to stand out for one head (a multiple of its query); it sits at, just before and
    just after the borders of pages, tiles of 32 and chunks of 256, as the first key and as the row's own.  Rows are
    single tokens (keys split over blocks and merged) and rows of a portion (one block per row).  The penalty's
    constants are small for the marked head, so that the far key wins against the near ones."""
    torch.manual_seed(3)
    heads, groups, dk, dv, page, context = 4, 2, 24, 40, 16, 530
    r1 = torch.tensor([0.4, 0.05, 1.0, 0.7]) if kind == "penalty" else None
    r2 = torch.tensor([0.5, 0.01, 0.2, 1.0]) if kind == "penalty" else None
    sink = torch.tensor([0.5, -1.0, 2.0, 0.0]) if kind == "sink_mixed" else None
    mix = (0.6 * torch.eye(heads) + 0.3 * torch.randn(heads, heads)) if kind == "sink_mixed" else None
    for special in (0, 1, 15, 16, 31, 32, 255, 256, 257, 511, 512, 529):
        keys = (torch.randn(context, groups, dk) * 0.3).to(dtype).float()
        values = torch.randn(context, groups, dv).to(dtype).float()
        q = torch.randn(1, heads, dk).to(dtype).float()
        keys[special, 0] = (q[0, 1] * 3.0).to(dtype).float()               # head 1 (group 0) looks at `special`
        k_cache, v_cache, table = _paged(keys, values, page, seed=special)
        for positions in ([context - 1], [special], list(range(special, min(context, special + 70)))):
            queries = q.expand(len(positions), heads, dk).contiguous()
            want = _plain_rows(queries, keys, values, positions, 0.9, r1, r2, sink, mix)
            for split in (True, False) if len(positions) == 1 else (None,):
                got = _attend(queries, k_cache, v_cache, table, positions, 0.9, dtype, r1, r2, sink, mix, split)
                limit = 3e-5 if dtype == torch.float32 else 3e-2
                assert float((got - want).abs().max()) <= limit * max(1.0, float(want.abs().max())), (special, positions[:3], split)
        if special > 40:   # the marked key carries the row: without it the row differs (the test would notice a lost key)
            unmarked = keys.clone()
            unmarked[special, 0] = 0.0
            other = _plain_rows(q, unmarked, values, [context - 1], 0.9, r1, r2, sink, mix)
            marked = _plain_rows(q, keys, values, [context - 1], 0.9, r1, r2, sink, mix)
            assert float((other - marked).abs().max()) > 0.05


def test_attention_many_heads_a_group_and_one_head_a_group():
    """Nine and seventeen query heads on one key/value head (more than one block of heads), and as many key/value heads
    as query heads, with the weights of every head mixed over the values of its own group."""
    torch.manual_seed(4)
    for heads, groups, dk, dv in ((9, 1, 12, 28), (34, 2, 16, 8), (5, 5, 20, 20), (6, 3, 8, 36)):
        context, page = 77, 8
        keys, values = torch.randn(context, groups, dk) * 0.5, torch.randn(context, groups, dv)
        q = torch.randn(context, heads, dk)
        sink, mix = torch.randn(heads), torch.randn(heads, heads) * 0.5
        r1, r2 = torch.rand(heads) + 0.1, torch.rand(heads) + 0.1
        k_cache, v_cache, table = _paged(keys, values, page, seed=heads)
        positions = list(range(context))
        got = _attend(q, k_cache, v_cache, table, positions, 0.7, torch.float32, sink=sink, mix=mix)
        want = _plain_rows(q, keys, values, positions, 0.7, sink=sink, table=mix)
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), (heads, groups, "mixed")
        got = _attend(q, k_cache, v_cache, table, positions, 0.7, torch.float32, r1=r1, r2=r2)
        want = _plain_rows(q, keys, values, positions, 0.7, r1, r2)
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), (heads, groups, "penalty")


def test_a_sink_alone_takes_weight_and_a_far_key_pays_the_penalty():
    """The first token of a sequence with a sink: its only key shares the softmax with the sink.  And the penalty at
    distance d is r1 ln(1 + r2 d): two equal keys at distances 0 and d get weights in the ratio (1 + r2 d)^r1."""
    keys, values = torch.ones(1, 1, 8), torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    q = torch.zeros(1, 2, 8)
    k_cache, v_cache, table = _paged(keys, values, 4)
    sink = torch.tensor([0.0, 1.0])
    got = _attend(q, k_cache, v_cache, table, [0], 1.0, torch.float32, sink=sink)
    for head in range(2):
        share = 1.0 / (1.0 + float(torch.exp(sink[head])))
        assert float((got[0, head] - values[0, 0] * share).abs().max()) <= 1e-6
    distance, r1, r2 = 300, torch.tensor([0.7]), torch.tensor([0.2])
    keys = torch.zeros(distance + 1, 1, 8)
    values = torch.zeros(distance + 1, 1, 4)
    values[0, 0, 0] = 1.0
    values[distance, 0, 1] = 1.0
    k_cache, v_cache, table = _paged(keys, values, 16)
    penalties = r1 * torch.log1p(r2 * torch.arange(distance, -1, -1.0))
    weights = torch.softmax(-penalties, 0)
    got = _attend(torch.zeros(1, 1, 8), k_cache, v_cache, table, [distance], 1.0, torch.float32, r1=r1, r2=r2)
    assert abs(float(got[0, 0, 0]) - float(weights[0])) <= 1e-6 and abs(float(got[0, 0, 1]) - float(weights[-1])) <= 1e-6
    assert abs(float(got[0, 0, 1] / got[0, 0, 0]) - (1.0 + 0.2 * distance) ** 0.7) <= 1e-3


def test_head_norm_bias_and_page_write():
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(5)
    for n_q, n_kv, dk, dv in ((4, 2, 24, 40), (3, 3, 10, 6), (5, 0, 36, 20)):
        rows, page, pages = 11, 4, 6
        width = n_q * dk + n_kv * (dk + dv) + 7                       # further columns (a gate) that the kernel leaves alone
        proj = torch.randn(2, rows, width)                           # two partial sums
        bias = torch.randn(n_q * dk + n_kv * (dk + dv))
        q_norm, k_norm = torch.rand(dk) + 0.5, torch.rand(dk) + 0.5
        slots = torch.randperm(page * pages)[:rows].to(torch.int32)
        slots[3] = -1                                                # a padding row writes nothing
        q_out = torch.empty(rows, n_q, dk, device="cuda")
        k_cache = torch.zeros(pages, max(n_kv, 1), page, dk, device="cuda")
        v_cache = torch.zeros(pages, max(n_kv, 1), page, dv, device="cuda")
        ops.head_norm_kv_write(proj.cuda(), bias.cuda(), q_norm.cuda(), k_norm.cuda() if n_kv else None, 1e-5,
                               slots.cuda() if n_kv else None, q_out, k_cache if n_kv else None, v_cache if n_kv else None,
                               n_q, n_kv, dk, dv)
        total = (proj[0] + proj[1])[:, :bias.shape[0]].double() + bias.double()
        want_q = plain.head_norm(total[:, :n_q * dk], n_q, q_norm.double(), 1e-5)
        assert float((q_out.cpu() - want_q).abs().max()) <= 1e-5
        if n_kv:
            want_k = plain.head_norm(total[:, n_q * dk:(n_q + n_kv) * dk], n_kv, k_norm.double(), 1e-5)
            want_v = total[:, (n_q + n_kv) * dk:].view(rows, n_kv, dv)
            for row in range(rows):
                slot = int(slots[row])
                if slot < 0:
                    continue
                assert float((k_cache[slot // page, :, slot % page].cpu() - want_k[row]).abs().max()) <= 1e-5
                assert float((v_cache[slot // page, :, slot % page].cpu() - want_v[row]).abs().max()) <= 1e-5
            written = sorted(int(slot) for slot in slots if slot >= 0)
            untouched = [slot for slot in range(page * pages) if slot not in written]
            assert float(k_cache.transpose(1, 2).reshape(page * pages, -1)[untouched].abs().max()) == 0.0


def test_norm_after_the_sum_embedding_and_cap():
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(6)
    rows, width = 7, 50
    for copy_dtype in (None, torch.bfloat16):
        x = torch.randn(rows, width)
        delta, bias, weight, extra = torch.randn(3, rows, width), torch.randn(width), torch.randn(width), torch.rand(rows)
        copy = None if copy_dtype is None else x.to(copy_dtype).cuda()
        source = x if copy is None else copy.float().cpu()
        total = 2.5 * x.double() + delta.sum(0).double() + bias.double() + extra.double()[:, None] * source.double()
        want = plain.norm(total, weight.double(), 1e-5)
        residual = x.cuda()
        ops.scaled_add_rmsnorm(residual, delta.cuda(), bias.cuda(), extra.cuda(), 2.5, weight.cuda(), 1e-5, copy)
        assert float((residual.cpu() - want).abs().max()) <= 1e-5 * float(want.abs().max())
        if copy is not None:
            assert torch.equal(copy.cpu(), residual.cpu().to(copy_dtype))
    table, positions_table = torch.randn(30, width), torch.randn(40, width)
    ids = torch.tensor([3, 29, 0, 3], dtype=torch.int32)
    positions = torch.tensor([0, 39, 17, 5], dtype=torch.int32)
    residual = torch.empty(4, width, device="cuda")
    ops.embedding_positions(table.cuda(), positions_table.cuda(), ids.cuda(), positions.cuda(), 0.25, residual, None)
    want = table[ids.long()] * 0.25 + positions_table[positions.long()]
    assert float((residual.cpu() - want).abs().max()) <= 1e-6
    values = torch.linspace(-90.0, 90.0, 1001)
    got = ops.softcap(values.cuda(), 30.0).cpu()
    assert float((got - 30.0 * torch.tanh(values.double() / 30.0)).abs().max()) <= 1e-5


def _mixture_case(experts, identity, top, ff, limit, shared, width, rows, seed, dtype=torch.float32):
    from llm_serving_engine_b200.parts.base import BuildContext
    from llm_serving_engine_b200.parts.moe import ClampedMoE

    mlp = moe(experts, identity, top, ff, limit, shared)
    generator = torch.Generator().manual_seed(seed)
    draw = lambda *shape, std=1.0: (torch.randn(*shape, generator=generator) * std).to(torch.bfloat16).float()
    weights = {"router": draw(experts + identity, width, std=4.0 / width ** 0.5), "correction": draw(experts + identity, std=0.2)}
    names = [f"e{index}." for index in range(experts)] + (["shared."] if shared else [])
    for name in names:
        size = shared[0] if name == "shared." else ff
        weights[name + "gate"], weights[name + "up"] = draw(size, width, std=1.5 / width ** 0.5), draw(size, width, std=1.5 / width ** 0.5)
        weights[name + "down"] = draw(width, size, std=1.0 / size ** 0.5)
    if shared:
        weights["shared.sg"] = draw(1, width, std=1.0 / width ** 0.5)
    x = draw(rows, width)
    want = plain.mixture(x.double(), {"p." + name: tensor.double() for name, tensor in weights.items()}, "p.", mlp)
    params = {"experts": experts, "identity": identity, "top": top, "ff": ff, "limit": limit,
              "shared": {"ff": shared[0], "limit": shared[1]} if shared else None}
    held = {name: tensor.cuda().to(dtype if tensor.dim() == 2 else torch.float32) for name, tensor in weights.items()}
    part = ClampedMoE(params, held, BuildContext(dtype, torch.device("cuda"), width, 0, 64))
    got = part.forward(x.cuda().to(dtype))
    from llm_serving_engine_b200.parts.linear import reduce_partials
    got = reduce_partials(got).float().cpu()
    if part.row_scale is not None:     # the identity experts' share, which the part leaves to the norm that follows
        got = got + part.row_scale.cpu()[:, None] * x
    return got, want, x, weights, mlp


@pytest.mark.parametrize("rows", [1, 5, 70])
def test_mixture_of_experts_against_the_plain_mixture(rows):
    """Few rows (the few-rows products and their partial sums) and many; identity experts, one expert, no shared
    expert, more chosen than real experts, odd sizes."""
    for case, (experts, identity, top, ff, limit, shared, width) in enumerate((
            (5, 2, 3, 40, 0.8, (56, 1.5), 72), (4, 0, 1, 24, 0.5, None, 64), (1, 3, 3, 18, 0.3, (10, 0.5), 102),
            (10, 3, 4, 48, 1.2, (80, 1.8), 128))):
        got, want, *_ = _mixture_case(experts, identity, top, ff, limit, shared, width, rows, seed=10 * rows + case)
        assert float((got - want).abs().max()) <= 3e-5 * float(want.abs().max()), (rows, case)


def test_router_choice_uses_the_correction_and_the_weights_do_not():
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(7)
    rows, width, outputs, identity, top = 40, 32, 9, 3, 4
    x, router = torch.randn(rows, width), torch.randn(outputs, width) * 0.5
    correction = torch.randn(outputs)                              # large: it changes most choices
    gate_w = torch.randn(width) * 0.2
    chosen = torch.empty(rows, top, dtype=torch.int32, device="cuda")
    logits = torch.zeros(3, rows, outputs + 3)                    # three partial sums, columns of padding behind the gate
    logits[:, :, :outputs + 1] = torch.cat([x @ router.t(), (x @ gate_w)[:, None]], dim=1) / 3.0
    weights, identity_weight, shared_gate = ops.moe_route(logits.cuda(), correction.cuda(), outputs, identity, top,
                                                          shared_gate=True, chosen=chosen)
    scores, want = plain.route(x.double(), router.double(), correction.double(), top)
    plain_choice = torch.topk(scores, top, dim=-1).indices
    assert not torch.equal(plain_choice.sort(-1).values, want.sort(-1).values)     # the correction matters in this case
    assert torch.equal(chosen.cpu().long().sort(-1).values, want.sort(-1).values)
    dense = torch.zeros(rows, outputs, dtype=torch.float64).scatter(1, want, scores.gather(1, want))
    assert float((weights.cpu() - dense[:, :outputs - identity]).abs().max()) <= 1e-5
    assert float((identity_weight.cpu() - dense[:, outputs - identity:].sum(-1)).abs().max()) <= 1e-5
    assert float((shared_gate.cpu() - torch.sigmoid(x.double() @ gate_w.double())).abs().max()) <= 1e-5


def test_tensor_core_attention_against_the_general_kernel():
    """Portions of several requests beside single tokens, pages scattered, groups of one, three (which does not divide a
    tile's 64 rows), eight and nine heads, with the penalty, the sink and the values of every group, whole and split
    by chunks: the tensor-core kernel against the float32-arithmetic kernel on the same bfloat16 inputs, and one far
    key that must be found."""
    from llm_serving_engine_b200.kernels import ops
    import numpy as np

    torch.manual_seed(8)
    page = 16
    for heads, groups, size in ((6, 3, 48), (3, 1, 32), (8, 8, 64), (16, 2, 128), (18, 2, 96), (6, 2, 64)):
        counts, firsts = [70, 1, 33, 1, 5], [300, 519, 0, 0, 63]
        contexts = [first + count for first, count in zip(firsts, counts)]
        pages_each = [-(-context // page) for context in contexts]
        pool_pages = sum(pages_each) + 3
        k_cache = (torch.randn(pool_pages, groups, page, size) * 0.5).to(torch.bfloat16).cuda()
        v_cache = torch.randn(pool_pages, groups, page, size).to(torch.bfloat16).cuda()
        order = torch.randperm(pool_pages).to(torch.int32)
        table = torch.full((len(counts), max(pages_each)), -1, dtype=torch.int32)
        cursor = 0
        for index, count in enumerate(pages_each):
            table[index, :count] = order[cursor:cursor + count]
            cursor += count
        total = sum(counts)
        q = (torch.randn(total, heads, size) * 0.5).to(torch.bfloat16)
        k_cache[int(table[0, 1]), groups - 1, 3] = (q[5, heads - 1] * 4.0).cuda()     # key 19 of request 0 stands out for the last head
        starts = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32).cuda()
        seg = torch.cat([torch.full((count,), index, dtype=torch.int32) for index, count in enumerate(counts)]).cuda()
        pos = torch.cat([torch.arange(first, first + count, dtype=torch.int32) for first, count in zip(firsts, counts)]).cuda()
        first_pos = torch.tensor(firsts, dtype=torch.int32).cuda()
        assert ops.attention_scored_mma_supported(size, size, heads, groups, torch.bfloat16)
        assert not ops.attention_scored_mma_supported(size, size + 16, heads, groups, torch.bfloat16)
        sink = torch.linspace(-1.0, 2.0, heads).cuda()
        r1, r2 = (torch.rand(heads) * 0.2).cuda(), (torch.rand(heads) * 0.5 + 0.01).cuda()
        for kind in ("plain", "penalty", "sink", "sink_cross"):
            extra = {"penalty": dict(r1=r1, r2=r2), "sink": dict(sink=sink), "sink_cross": dict(sink=sink, cross=True)}.get(kind, {})
            slots = groups if kind == "sink_cross" else 1
            for split in (False, True):
                for out_dtype in (torch.bfloat16, torch.float32):
                    want = torch.empty(total, heads, slots, size, dtype=out_dtype, device="cuda")
                    got = torch.full_like(want, float("nan"))
                    ops.attention_scored(q.cuda(), k_cache, v_cache, want, table.cuda(), seg, pos, 0.3, split=split,
                                         tensor_cores=False, **extra)
                    ops.attention_scored(q.cuda(), k_cache, v_cache, got, table.cuda(), seg, pos, 0.3, split=split,
                                         segment_start=starts, segment_first_position=first_pos, **extra)
                    error = float((got.float() - want.float()).abs().max())
                    assert error <= 2e-2 * max(1.0, float(want.float().abs().max())), (heads, groups, size, kind, split, error)


@pytest.mark.parametrize("rows", [5, 70, 300])
def test_mixture_of_experts_in_bfloat16_both_ways_through_the_experts(rows, monkeypatch):
    """bfloat16: few rows take every expert's product (partial sums), many rows are grouped by expert for the grouped
    product; both against the plain mixture, and the two ways against each other on the same rows.  One case has an
    expert that no row chooses and rows whose choices are all identity experts."""
    from llm_serving_engine_b200.parts import moe as moe_part

    for case, (experts, identity, top, ff, limit, shared, width) in enumerate((
            (5, 2, 3, 40, 0.8, (56, 1.5), 72), (4, 0, 1, 24, 0.5, None, 64), (2, 6, 2, 16, 0.3, (8, 0.5), 104),
            (10, 3, 4, 48, 1.2, (80, 1.8), 128))):
        got, want, *_ = _mixture_case(experts, identity, top, ff, limit, shared, width, rows, seed=10 * rows + case,
                                      dtype=torch.bfloat16)
        scale = float(want.abs().max())
        assert float((got - want).abs().max()) <= 3e-2 * scale, (rows, case)
        monkeypatch.setattr(moe_part, "GROUPED_FROM_ROWS", 1 if rows < moe_part.GROUPED_FROM_ROWS else 10 ** 9)
        other, *_ = _mixture_case(experts, identity, top, ff, limit, shared, width, rows, seed=10 * rows + case,
                                  dtype=torch.bfloat16)
        monkeypatch.undo()
        assert float((got - other).abs().max()) <= 3e-2 * scale, (rows, case, "the two ways")


def test_rows_grouped_by_expert_have_places_of_their_own():
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(9)
    tokens, top, experts = 333, 3, 7
    chosen = torch.stack([torch.randperm(experts + 2)[:top] for _ in range(tokens)]).to(torch.int32)   # ids 7, 8: identity
    chosen[:, 0][chosen[:, 0] == 4] = 5                                                               # expert 4 is rarer
    segment = torch.zeros(tokens, dtype=torch.int32)
    segment[-5:] = -1                                                                                 # padding rows
    row_of, offsets = ops.moe_group_rows(chosen.cuda(), experts, segment.cuda())
    row_of, offsets = row_of.cpu(), offsets.cpu()
    live = chosen[:-5]
    counts = torch.tensor([(live == e).sum() for e in range(experts)])
    assert torch.equal(offsets.long(), counts.cumsum(0))
    assert bool((row_of[-5:] == -1).all()) and bool((row_of[:-5][live >= experts] == -1).all())
    placed = row_of[:-5][live < experts]
    assert sorted(placed.tolist()) == list(range(int(counts.sum())))                                   # every place once
    firsts = torch.cat([torch.zeros(1, dtype=torch.long), counts.cumsum(0)[:-1]])
    for e in range(experts):
        rows = row_of[:-5][live == e]
        assert bool(((rows >= firsts[e]) & (rows < firsts[e] + counts[e])).all())


def test_tcgen05_attention_against_the_general_kernel():
    """Prompt portions of several requests (one from position 0, one behind a long prefix, one of a single token, one
    that ends inside a tile), pages scattered, heads of 64 and 128 in groups of one, two and eight, with the penalty,
    the sink and the values of every group: the tcgen05 kernel against the float32-arithmetic kernel on the same
    bfloat16 inputs, and one far key that must be found."""
    from llm_serving_engine_b200.kernels import ops
    import numpy as np

    torch.manual_seed(11)
    page = 16
    for heads, groups, size in ((6, 2, 64), (8, 1, 128), (3, 3, 128)):
        counts, firsts = [300, 1, 129, 140], [0, 77, 500, 1000]
        contexts = [first + count for first, count in zip(firsts, counts)]
        pages_each = [-(-context // page) for context in contexts]
        pool_pages = sum(pages_each) + 3
        k_cache = (torch.randn(pool_pages, groups, page, size) * 0.5).to(torch.bfloat16).cuda()
        v_cache = torch.randn(pool_pages, groups, page, size).to(torch.bfloat16).cuda()
        order = torch.randperm(pool_pages).to(torch.int32)
        table = torch.full((len(counts), max(pages_each)), -1, dtype=torch.int32)
        cursor = 0
        for index, count in enumerate(pages_each):
            table[index, :count] = order[cursor:cursor + count]
            cursor += count
        total = sum(counts)
        q = (torch.randn(total, heads, size) * 0.5).to(torch.bfloat16)
        k_cache[int(table[3, 1]), groups - 1, 3] = (q[total - 5, heads - 1] * 4.0).cuda()   # key 19 of the last request, far back
        starts = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32).cuda()
        seg = torch.cat([torch.full((count,), index, dtype=torch.int32) for index, count in enumerate(counts)]).cuda()
        pos = torch.cat([torch.arange(first, first + count, dtype=torch.int32) for first, count in zip(firsts, counts)]).cuda()
        first_pos = torch.tensor(firsts, dtype=torch.int32).cuda()
        sink = torch.linspace(-1.0, 2.0, heads).cuda()
        r1, r2 = (torch.rand(heads) * 0.2).cuda(), (torch.rand(heads) * 0.5 + 0.01).cuda()
        for kind in ("plain", "penalty", "sink", "sink_cross"):
            extra = {"penalty": dict(r1=r1, r2=r2), "sink": dict(sink=sink), "sink_cross": dict(sink=sink, cross=True)}.get(kind, {})
            slots = groups if kind == "sink_cross" else 1
            want = torch.empty(total, heads, slots, size, dtype=torch.float32, device="cuda")
            got = torch.full((total, heads, slots, size), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.attention_scored(q.cuda(), k_cache, v_cache, want, table.cuda(), seg, pos, 0.3, tensor_cores=False, **extra)
            ops.attention_scored_tc(q.cuda(), k_cache, v_cache, got, table.cuda(), starts, first_pos, 0.3, **extra)
            assert ops.attention_tc_status() == 0
            error = float((got.float() - want).abs().max())
            assert error <= 2e-2 * max(1.0, float(want.abs().max())), (heads, groups, size, kind, error)


def test_long_prompts_take_the_tcgen05_kernel_and_agree_with_the_plain_model():
    """Heads of 64 and 128: prompts of 128 rows and more run on the tcgen05 kernel in bfloat16 (whole, and in portions
    behind a prefix), shorter steps on the mma.sync kernel; the logits agree with the plain model either way."""
    from llm_serving_engine_b200.models import load_model

    name = "tensor_core_sizes"
    CONFIGS[name] = model([attention2(heads=6, kv_heads=3, dim=64, vdim=64), attention(heads=2, kv_heads=1, dim=128, vdim=128),
                           attention(heads=4, kv_heads=1, dim=128, vdim=128, kv_from=1, mlp=None),
                           attention2(heads=2, kv_heads=2, dim=128, vdim=128, mlp=None)], width=96, positions=700)
    engine_model = load_model(folder_of(name), dtype="bfloat16")
    assert engine_model.launch_signature([300]) == (("tcgen05",),) and engine_model.launch_signature([100, 20]) == ()
    requests = some_requests(name, [330, 140], seed=13)
    got = replay(name, "bfloat16", helpers.trace_whole(requests), helpers.max_tokens_for(requests))
    compare(name, "bfloat16", requests, got, "whole prompts on tcgen05")
    got = replay(name, "bfloat16", helpers.trace_portions(requests, (150, 130, 20, 2)), helpers.max_tokens_for(requests))
    compare(name, "bfloat16", requests, got, "portions on tcgen05")
