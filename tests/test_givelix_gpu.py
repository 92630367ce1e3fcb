"""The Givelix design through the engine against the plain implementation (``tests/plain/givelix_plain.py``):
every mixer alone and together, whole prompts, decoding through the cache and the state, portions down to two
tokens, mixed batches with pages and state slots that are used again, other sizes, both precisions, and greedy
generation through ``LLMEngine``."""
import json
import random
import tempfile
from pathlib import Path

import numpy as np
import pytest
import torch

import helpers
from plain import givelix_plain as plain

pytestmark = pytest.mark.gpu

ROT = {"base": 10000.0, "dims": 8}
ROT_SCALED = {"base": 50000.0, "dims": 12, "scaling": {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}}


def lightning(heads=3, dim=24, vdim=40, decay=(0.5, 0.97, 0.9995), mlp=None):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}, "mlp": mlp}


def latent(heads=3, dim=24, rot_dim=8, vdim=20, kv_rank=40, q_rank=36, rot=ROT, kv_from=None, mlp=None):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": 1.7 / (dim + rot_dim) ** 0.5, "rot": dict(rot)}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def latent2(heads=5, dim=16, rot_dim=12, vdim=24, kv_rank=56, rot=ROT_SCALED, mlp=None):
    return {"type": "latent_attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "scale": 2.1 / (dim + rot_dim) ** 0.5, "rot": dict(rot)}}


def model(layers, width=72, vocab=211, streams=3, mult=0.4, logit_scale=0.7):
    config = {"architecture": "Givelix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": 1e-5},
              "residual_mult": mult, "logit_scale": logit_scale}
    if streams is not None:
        config["streams"] = streams
    return config


DENSE = {"kind": "dense", "ff": 104}
CONFIGS = {
    "lightning_only": model([lightning(mlp=DENSE), lightning(heads=1, dim=40, vdim=8, decay=(0.8,))]),
    "latent_only": model([latent(mlp=DENSE), latent(kv_from=0)], streams=None),
    "latent2_only": model([latent2(), latent2(heads=2, dim=8, rot_dim=4, vdim=8, kv_rank=24,
                                          rot={"base": 100.0, "dims": 4}, mlp=DENSE)], streams=1),
    "all_kinds": model([latent(mlp=DENSE), lightning(), latent(kv_from=0, heads=2, dim=16, vdim=8, q_rank=20, mlp=DENSE),
                        latent2(mlp=DENSE), lightning(heads=2, dim=36, vdim=16, decay=(0.6, 0.999), mlp=DENSE), latent2()],
                       width=80, streams=4),
    # values that many models make equal or one: one head, one stream with tables, dim = vdim = rank, no layer scale
    "equal_sizes": model([latent(heads=1, dim=16, rot_dim=16, vdim=16, kv_rank=16, q_rank=16, rot={"base": 300.0, "dims": 16}),
                          lightning(heads=1, dim=32, vdim=32, decay=(0.9,), mlp=DENSE)], width=64, streams=1, mult=1.0,
                         logit_scale=1.0),
    # sizes that no vector load, tensor-core tile or few-rows product takes: every kernel's plain path
    "odd_sizes": model([lightning(heads=2, dim=48, vdim=20, decay=(0.7, 0.99)),
                        latent(heads=5, dim=20, rot_dim=6, vdim=12, kv_rank=36, q_rank=30, rot={"base": 777.0, "dims": 6},
                               mlp={"kind": "dense", "ff": 90}),
                        latent2(heads=3, dim=10, rot_dim=6, vdim=14, kv_rank=22,
                                rot={"base": 1000.0, "dims": 6, "scaling": {"factor": 3.0, "original": 40, "fast": 8.0, "slow": 1.0}},
                                mlp={"kind": "dense", "ff": 50}),
                        # a reader of a cache that is not the first layer's, with other heads and sizes of its own
                        latent(heads=9, dim=8, rot_dim=6, vdim=10, kv_rank=36, q_rank=14, rot={"base": 777.0, "dims": 6}, kv_from=1)],
                       width=102, vocab=333, streams=2),
}
NO_LAYER_SCALE = {"equal_sizes"}
# bfloat16: the random models are made with large gains so that every mechanism matters; their rounding noise is
# a few hundredths of the logits, a wrong mechanism moves them by tenths and more (and float32 pins the rest)
RMS_LIMIT = {"float32": 1.0e-5, "bfloat16": 1.0e-1}
_MODELS: dict = {}


def folder_of(name: str):
    if name not in _MODELS:
        holder = tempfile.TemporaryDirectory(prefix=f"givelix_{name}_")
        plain.write_model(holder.name, CONFIGS[name], seed=11 + len(_MODELS), layer_scale=name not in NO_LAYER_SCALE)
        _MODELS[name] = (holder, Path(holder.name), plain.load_folder(holder.name))
    return _MODELS[name][1]


def reference(name: str, tokens):
    folder_of(name)
    config, weights = _MODELS[name][2]
    return plain.forward_full(config, weights, tokens).to(torch.float32)


def replay(name: str, dtype: str, steps, max_tokens: int, page: int = 16, max_requests: int = 4):
    from llm_serving_engine_b200.engine.trace_replay import replay as run

    with tempfile.TemporaryDirectory(prefix="givelix_out_") as out:
        run(folder_of(name), dtype, out, max_tokens, [json.dumps(step) for step in steps], block_size=page,
            max_requests=max_requests)
        return helpers.collect(steps, Path(out))


def compare(name, dtype, requests, got, what):
    for rid, tokens in requests.items():
        want = reference(name, tokens)
        assert got[rid].shape == want.shape, f"{what}: {rid}: shape {tuple(got[rid].shape)} against {tuple(want.shape)}"
        centred = want - want.mean(-1, keepdim=True)
        per_row = (got[rid] - want).double().pow(2).mean(-1).sqrt() / centred.double().pow(2).mean().sqrt()
        worst = float(per_row.max())
        assert worst <= RMS_LIMIT[dtype], (f"{what}: {name} {dtype} request {rid}: row error / logit size {worst:.2e} at "
                                           f"position {int(per_row.argmax())}, first above the limit "
                                           f"{int((per_row > RMS_LIMIT[dtype]).nonzero()[0])}")


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_then_token_by_token(name, dtype):
    """Decoding reads the pages and the state that the prompt step left; the single tokens are replayed from a
    captured graph, whose warm-up run must leave the state as it was."""
    requests = some_requests(name, [40, 9, 3], seed=6)
    got = replay(name, dtype, helpers.trace_tail_decode(requests, tail=24), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "tail decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_of_changing_size(dtype):
    requests = some_requests("all_kinds", [150, 33], seed=7)
    for sizes in ((7, 2, 13, 3, 2, 31, 5, 16, 2, 64, 17), (2,), (16, 16, 1, 15, 17)):
        got = replay("all_kinds", dtype, helpers.trace_portions(requests, sizes), helpers.max_tokens_for(requests))
        compare("all_kinds", dtype, requests, got, f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 8])
def test_mixed_batches_reuse_pages_and_state_slots(dtype, page):
    """Nine requests through four state slots and a pool sized for the live ones only: a slot's state must be
    zero for its next request, and a page's old rows must not be read."""
    requests = some_requests("all_kinds", [61, 5, 90, 33, 2, 47, 130, 18, 64], seed=8)
    steps, peak = helpers.trace_mixed(requests, seed=3, max_live=4)
    got = replay("all_kinds", dtype, steps, peak, page=page)
    compare("all_kinds", dtype, requests, got, "mixed")


def test_a_batch_gives_what_each_request_gives_alone():
    requests = some_requests("all_kinds", [37, 12, 80, 5], seed=9)
    steps, peak = helpers.trace_mixed(requests, seed=4, max_live=4)
    together = replay("all_kinds", "float32", steps, peak)
    for rid, tokens in requests.items():
        alone = replay("all_kinds", "float32", helpers.trace_whole({rid: tokens}), helpers.max_tokens_for({rid: tokens}))
        assert float((together[rid] - alone[rid]).abs().max()) <= 2e-5 * float(alone[rid].abs().max())


def test_long_decoding_carries_the_state_and_crosses_key_chunks():
    """600 single tokens after a short prompt: the lightning state is carried through 600 graph replays, the latent
    attention's keys pass the borders of its tiles (32), chunks (256) and many pages."""
    requests = some_requests("all_kinds", [610], seed=10)
    got = replay("all_kinds", "float32", helpers.trace_tail_decode(requests, tail=600), 640)
    compare("all_kinds", "float32", requests, got, "long decoding")


def test_greedy_generation_through_the_engine_and_its_scheduler():
    """More requests than the scheduler keeps live, prompts cut into portions: every request's greedy tokens equal
    the plain implementation's (float32; a request whose top two logits are closer than the arithmetic's noise is
    skipped from that token on)."""
    from llm_serving_engine_b200.config import CacheConfig, SchedulerConfig
    from llm_serving_engine_b200.engine.llm_engine import LLMEngine
    from llm_serving_engine_b200.sampling.sampler import GenerationConfig
    from llm_serving_engine_b200.models import load_model

    name = "all_kinds"
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
def _latent_plain(q, rows, positions, scale, rank, sink, window=0):
    out = torch.zeros(q.shape[0], q.shape[1], rank, dtype=torch.float64)
    for t, pos in enumerate(positions):
        first = max(0, pos + 1 - window) if window else 0
        keys = rows[first:pos + 1].double()
        scores = torch.einsum("hd,jd->hj", q[t].double(), keys) * scale
        top = scores.max(-1, keepdim=True).values
        if sink is not None:
            top = torch.maximum(top, sink.double()[:, None])
        weights = torch.exp(scores - top)
        total = weights.sum(-1, keepdim=True)
        if sink is not None:
            total = total + torch.exp(sink.double()[:, None] - top)
        out[t] = (weights / total) @ keys[:, :rank]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("use_sink", [False, True])
def test_latent_attention_finds_one_far_key_at_every_border(dtype, use_sink):
    """One key among hundreds is made to stand out (its row is a multiple of the query); it sits at, just before and
    just after the borders of pages, tiles of 32 and chunks of 256, as the first key and as the row's own.  Rows are
    single tokens (keys split over blocks and merged) and rows of a portion (one block per row)."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(3)
    heads, rank, rot, page = 3, 40, 8, 16
    width, context = rank + rot, 530
    pages = -(-context // page)
    order = torch.randperm(pages + 5)[:pages].to(torch.int32)          # pages scattered over a larger pool
    for special in (0, 15, 16, 31, 32, 255, 256, 257, 511, 512, 529):
        rows = torch.randn(context, width) * 0.3
        q = torch.randn(1, heads, width)
        rows[special] = q[0, 1] * 2.0                                    # head 1 looks at `special`
        rows, q = rows.to(dtype).float(), q.to(dtype).float()
        pool = torch.full((pages + 5, page, width), float("nan"))      # unowned pages hold anything
        for logical in range(pages):
            chunk = rows[logical * page:(logical + 1) * page]
            pool[int(order[logical])].zero_()
            pool[int(order[logical]), :chunk.shape[0]] = chunk
        sink = torch.tensor([0.5, -1.0, 2.0]) if use_sink else None
        for positions in ([context - 1], [special], list(range(special, min(context, special + 70)))):
            count = len(positions)
            queries = q.expand(count, heads, width).contiguous()
            want = _latent_plain(queries, rows, positions, 0.9, rank, sink)
            got = torch.empty(count, heads, rank, dtype=dtype, device="cuda")
            ops.latent_attention(queries.to(dtype).cuda(), pool.to(dtype).cuda(), got, order.view(1, -1).cuda(),
                                 torch.zeros(count, dtype=torch.int32, device="cuda"),
                                 torch.tensor(positions, dtype=torch.int32, device="cuda"), 0.9,
                                 None if sink is None else sink.cuda(), split=count == 1)
            limit = 2e-5 if dtype == torch.float32 else 2e-2
            assert float((got.float().cpu() - want).abs().max()) <= limit, (special, positions[:3], count)


def test_tensor_core_latent_attention_against_the_general_kernel():
    """Portions of several requests beside single tokens, pages scattered, odd numbers of heads, with and without a
    sink, whole and split by chunks: the tensor-core kernel against the float32-arithmetic kernel on the same
    bfloat16 inputs, and one far key that must be found."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(8)
    page = 16
    for heads, rank, rot in ((3, 64, 16), (16, 128, 32), (40, 192, 16), (6, 24, 8)):
        width = rank + rot
        counts, firsts = [70, 1, 33, 1, 5], [300, 519, 0, 0, 63]
        contexts = [first + count for first, count in zip(firsts, counts)]
        pages_each = [-(-context // page) for context in contexts]
        pool = (torch.randn(sum(pages_each) + 3, page, width) * 0.5).to(torch.bfloat16).cuda()
        order = torch.randperm(sum(pages_each) + 3).to(torch.int32)
        table = torch.full((len(counts), max(pages_each)), -1, dtype=torch.int32)
        cursor = 0
        for index, count in enumerate(pages_each):
            table[index, :count] = order[cursor:cursor + count]
            cursor += count
        total = sum(counts)
        q = (torch.randn(total, heads, width) * 0.5).to(torch.bfloat16)
        pool[int(table[0, 1]), 3] = (q[5, heads - 1] * 4.0).cuda()          # key 19 of request 0 stands out for one head
        starts = torch.tensor([0] + list(np.cumsum(counts)), dtype=torch.int32).cuda()
        seg = torch.cat([torch.full((count,), index, dtype=torch.int32) for index, count in enumerate(counts)]).cuda()
        pos = torch.cat([torch.arange(first, first + count, dtype=torch.int32) for first, count in zip(firsts, counts)]).cuda()
        first_pos = torch.tensor(firsts, dtype=torch.int32).cuda()
        for sink in (None, torch.linspace(-1.0, 2.0, heads).cuda()):
            for split in (False, True):
                want = torch.empty(total, heads, rank, dtype=torch.bfloat16, device="cuda")
                got = torch.empty_like(want)
                ops.latent_attention(q.cuda(), pool, want, table.cuda(), seg, pos, 0.3, sink, split=split, tensor_cores=False)
                ops.latent_attention(q.cuda(), pool, got, table.cuda(), seg, pos, 0.3, sink, split=split,
                                     segment_start=starts, segment_first_position=first_pos)
                assert ops.latent_attention_mma_supported(width, rank, torch.bfloat16) == (rank % 8 == 0 and width % 16 == 0)
                error = float((got.float() - want.float()).abs().max())
                assert error <= 2e-2 * max(1.0, float(want.float().abs().max())), (heads, rank, rot, sink is not None, split, error)


def test_latent_attention_window_edges():
    """The kernel's window parameter: the key just inside the window is seen, the one just outside is not."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(4)
    heads, rank, rot, page, context, window = 2, 24, 8, 8, 300, 37
    width = rank + rot
    rows = torch.randn(context, width) * 0.3
    q = torch.randn(1, heads, width)
    pool = rows.view(-1, page, width).contiguous() if context % page == 0 else None
    if pool is None:
        pool = torch.zeros(-(-context // page) * page, width)
        pool[:context] = rows
        pool = pool.view(-1, page, width)
    table = torch.arange(pool.shape[0], dtype=torch.int32).view(1, -1)
    for pos in (window - 2, window - 1, window, 255, 256, 299):
        for offset in (window - 1, window):          # the last key inside, the first outside
            if pos - offset < 0:
                continue
            marked = rows.clone()
            marked[pos - offset] = q[0, 0] * 3.0
            marked_pool = pool.clone().view(-1, width)
            marked_pool[pos - offset] = marked[pos - offset]
            want = _latent_plain(q, marked, [pos], 1.0, rank, None, window)
            got = torch.empty(1, heads, rank, device="cuda")
            ops.latent_attention(q.cuda(), marked_pool.view(-1, page, width).cuda(), got, table.cuda(),
                                 torch.zeros(1, dtype=torch.int32, device="cuda"),
                                 torch.tensor([pos], dtype=torch.int32, device="cuda"), 1.0, None, window=window)
            assert float((got.cpu() - want).abs().max()) <= 2e-5, (pos, offset)


def test_linear_attention_scan_against_the_recurrence():
    """Odd sizes (dim beyond one thread's 32 rows, columns beyond one block), two requests of unequal length from
    non-zero states in slots that are not in order, decays from fast to almost none."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(5)
    for heads, dim, vdim in ((2, 24, 40), (3, 72, 136), (1, 130, 8)):
        width = heads * (2 * dim + 2 * vdim)
        counts, slots = [19, 1, 150], [2, 0, 3]
        proj = torch.randn(sum(counts), width)
        decay = torch.tensor([0.3, 0.95, 0.9999][:heads])
        state = torch.randn(4, heads, dim, vdim) * 0.5
        want_state = state.double().clone()
        want = torch.zeros(sum(counts), heads * vdim, dtype=torch.float64)
        row = 0
        for count, slot in zip(counts, slots):
            for t in range(row, row + count):
                z = proj[t].double()
                act = z * torch.sigmoid(z)
                q = act[:heads * dim].view(heads, dim)
                k = act[heads * dim:2 * heads * dim].view(heads, dim)
                v = act[2 * heads * dim:2 * heads * dim + heads * vdim].view(heads, vdim)
                for h in range(heads):
                    want_state[slot, h] = float(decay[h]) * want_state[slot, h] + torch.outer(k[h], v[h])
                    want[t, h * vdim:(h + 1) * vdim] = want_state[slot, h].t() @ q[h]
            row += count
        starts = torch.tensor([0, 19, 20, 170, 170], dtype=torch.int32).cuda()       # a fourth, empty request
        for chunked in (False, True):      # row by row, and in chunks of 64 rows scanned side by side (19, 1, 64 + 64 + 22)
            got = torch.empty(sum(counts), heads * vdim, device="cuda")
            device_state = state.cuda()
            ops.linear_attention_scan(proj.cuda(), 0, heads * dim, 2 * heads * dim, decay.cuda(), device_state, starts,
                                      torch.tensor(slots + [1], dtype=torch.int32).cuda(), got, heads, dim, vdim, "silu",
                                      chunked=chunked)
            scale = float(want.abs().max())
            assert float((got.cpu() - want).abs().max()) <= 2e-5 * scale, (heads, dim, vdim, chunked)
            assert float((device_state.cpu() - want_state).abs().max()) <= 2e-5 * float(want_state.abs().max())
            assert torch.equal(device_state[1].cpu(), state[1])                  # the empty request's slot is untouched


def test_residual_copies_update_and_norm():
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(6)
    rows, copies, width = 9, 3, 50
    x = torch.randn(rows, copies, width)
    delta = torch.randn(2, rows, width)              # two partial sums
    scale, mix = torch.rand(width) + 0.5, torch.randn(copies, copies)
    write, read, weight = torch.randn(copies), torch.randn(copies), torch.randn(width)
    y = (delta[0] + delta[1]).double() * 0.3 * scale.double()
    new = torch.einsum("sr,tsw->trw", mix.double(), x.double()) + write.double()[None, :, None] * y[:, None, :]
    u = torch.einsum("r,trw->tw", read.double(), new)
    want = u / torch.sqrt(u.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double()
    device_x = x.view(rows, -1).cuda()
    got = torch.empty(rows, width, device="cuda")
    ops.streams_update_rmsnorm(device_x, copies, delta.cuda(), scale.cuda(), 0.3, mix.cuda(), write.cuda(), read.cuda(),
                               weight.cuda(), 1e-5, got)
    assert float((got.cpu() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert float((device_x.cpu().view(rows, copies, width) - new).abs().max()) <= 1e-5 * float(new.abs().max())
    # chosen rows only, nothing written back, the copies summed
    picked = torch.tensor([7, 2], dtype=torch.int32)
    before = device_x.clone()
    got = torch.empty(2, width, device="cuda")
    ops.streams_update_rmsnorm(device_x, copies, None, None, 1.0, None, None, None, weight.cuda(), 1e-5, got,
                               rows=picked.cuda(), write_back=False)
    total = new[picked.long()].sum(1)
    want = total / torch.sqrt(total.pow(2).mean(-1, keepdim=True) + 1e-5) * weight.double()
    assert float((got.cpu() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert torch.equal(before, device_x)


def test_rotation_with_scaled_frequencies_reaches_the_cache():
    """The rotated shared key part as the prepare kernel writes it, at positions in the thousands, against the plain
    rotation with the same scaled frequencies."""
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.parts.latent_attention import rotary_frequencies

    torch.manual_seed(7)
    rank, rot = 24, 12
    freq, factor = rotary_frequencies(ROT_SCALED)
    plain_freq, plain_factor = plain.rotary_frequencies(ROT_SCALED)
    assert factor == plain_factor and float((freq - plain_freq).abs().max()) == 0.0
    assert float((freq / plain.rotary_frequencies({"base": 50000.0, "dims": 12})[0]).min()) < 0.3    # the scaling acts
    positions = torch.tensor([0, 1, 63, 64, 1000, 4097, 9999], dtype=torch.int32)
    proj = torch.randn(len(positions), rank + rot)
    norm = torch.rand(rank) + 0.5
    cache = torch.zeros(2, 8, rank + rot, device="cuda")
    slots = torch.tensor([3, 9, 0, 15, 7, 8, 12], dtype=torch.int32)
    ops.latent_prepare(proj.cuda(), positions.cuda(), slots.cuda(), 1e-5, kv_off=0, rank=rank, kv_norm=norm.cuda(),
                       rot=rot, rot_dims=12, freq=freq.cuda(), rot_factor=factor, cache=cache)
    want_latent = plain.plain_norm(proj[:, :rank].double(), norm.double(), 1e-5)
    want_shared = plain.rotate(proj[:, rank:].double(), positions, ROT_SCALED)
    got = cache.view(16, -1).cpu()[slots.long()]
    assert float((got[:, :rank] - want_latent).abs().max()) <= 1e-5
    assert float((got[:, rank:] - want_shared).abs().max()) <= 1e-5
