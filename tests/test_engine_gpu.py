"""The engine against the plain implementation under every way of cutting the work."""

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain
from tests.plain import tiny_models

pytestmark = pytest.mark.gpu

CONFIGS = {"A": (tiny_models.TINY_A, 0), "B": (tiny_models.TINY_B, 1), "C": (tiny_models.TINY_C, 2),
           "D": (tiny_models.TINY_D, 3), "E": (tiny_models.TINY_E, 4),
           # A with matrices fifteen times as large: with the usual N(0, 0.02) and a tied head, greedy
           # decoding of A only repeats the prompt's last token, which no test of generation can use
           "A_sharp": (tiny_models.TINY_A, 5)}
WEIGHT_OPTIONS = {"A_sharp": dict(linear_std=0.3)}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for tag, (cfg, seed) in CONFIGS.items():
        out[tag] = helpers.make_folder(tmp_path_factory.mktemp("tiny_" + tag), cfg, seed,
                                       **WEIGHT_OPTIONS.get(tag, {}))
    return out


@pytest.fixture(scope="module")
def engines(folders):
    from enginekernel_b200 import Engine
    cache = {}

    def get(tag, dtype):
        if (tag, dtype) not in cache:
            cache[(tag, dtype)] = Engine(folders[tag], dtype, max_tokens=4096, max_batch=8)
        return cache[(tag, dtype)]
    return get


@pytest.fixture(scope="module")
def plains(folders):
    return {tag: helpers.plain_model(folders[tag]) for tag in folders}


def lengths_for(tag):
    limit = CONFIGS[tag][0]["max_position_embeddings"]
    return [n for n in (1, 7, 33, 64, 65, 100, 200) if n <= limit]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_each_request_alone_and_whole(engines, plains, tag, dtype):
    cfg = CONFIGS[tag][0]
    eng = engines(tag, dtype)
    for k, n in enumerate(lengths_for(tag)):
        ids = tiny_models.random_prompts(cfg, [n], seed=40 + k)[0]
        err = helpers.rel_err(helpers.whole(eng, ids), plain.logits(plains[tag], ids))
        assert err <= helpers.TOL[dtype], f"{tag} {dtype} length {n}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_last_32_tokens_one_by_one(engines, plains, tag, dtype):
    cfg = CONFIGS[tag][0]
    eng = engines(tag, dtype)
    n = min(100, cfg["max_position_embeddings"])
    ids = tiny_models.random_prompts(cfg, [n], seed=77)[0]
    want = plain.logits(plains[tag], ids)
    got = helpers.tail_one_by_one(eng, ids, 32)
    err = helpers.rel_err(got, want)
    assert err <= helpers.TOL[dtype], f"{tag} {dtype}: {err:.3e}"
    if dtype == "float32":
        assert helpers.rel_err(got, helpers.whole(eng, ids)) <= 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["A", "B", "C", "D", "E"])
def test_unequal_batches_one_after_another(engines, plains, tag, dtype):
    """Batches of unequal lengths whose shorter requests end earlier; three batches in a
    row on an engine with few slots, so that slots and pages are used again."""
    cfg = CONFIGS[tag][0]
    eng = engines(tag, dtype)
    limit = cfg["max_position_embeddings"]
    shapes = [((5, 9, 13), (3, 9, 1)), ((1, 70, 31, 16), (1, 64, 20, 16)), ((66, 2, 40), (65, 1, 8))]
    for k, (lens, heads) in enumerate(shapes):
        lens = [min(n, limit) for n in lens]
        heads = [min(h, n) for h, n in zip(heads, lens)]
        seqs = tiny_models.random_prompts(cfg, lens, seed=200 + k)
        got = helpers.batch_then_steps(eng, seqs, heads)
        for ids, g in zip(seqs, got):
            err = helpers.rel_err(g, plain.logits(plains[tag], ids))
            assert err <= helpers.TOL[dtype], f"{tag} {dtype} batch {k} len {len(ids)}: {err:.3e}"
    assert eng.cache.book.open_slots() == []
    assert eng.cache.free_tokens() == eng.cache.num_pages * 64


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_of_a_sequence(engines, plains, dtype):
    """Positions 0, 1, 2 fed one by one from an empty slot."""
    tag = "B"
    cfg = CONFIGS[tag][0]
    eng = engines(tag, dtype)
    ids = tiny_models.random_prompts(cfg, [4], seed=5)[0]
    got = helpers.tail_one_by_one(eng, ids, tail=3)
    assert helpers.rel_err(got, plain.logits(plains[tag], ids)) <= helpers.TOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(engines, plains, dtype):
    """Hundreds of single-token steps across many page boundaries."""
    tag = "C"
    cfg = CONFIGS[tag][0]
    eng = engines(tag, dtype)
    ids = tiny_models.random_prompts(cfg, [700], seed=9)[0]
    got = helpers.tail_one_by_one(eng, ids, tail=690)
    err = helpers.rel_err(got, plain.logits(plains[tag], ids))
    assert err <= helpers.TOL[dtype], f"{err:.3e}"


def test_padding_and_batch_mates_change_nothing(engines):
    """32-bit logits of a request are the same alone and among others, bit for bit in
    the matrix products and within rounding in attention."""
    eng = engines("B", "float32")
    cfg = CONFIGS["B"][0]
    seqs = tiny_models.random_prompts(cfg, [17, 40, 3], seed=31)
    alone = [helpers.whole(eng, s) for s in seqs]
    together = helpers.batch_then_steps(eng, seqs, [len(s) for s in seqs])
    for a, t in zip(alone, together):
        assert helpers.rel_err(t, a) <= 1e-6


def check_tokens_against_plain(model, prompt, tokens, dtype):
    """32-bit: the plain arg-max at every position.  bfloat16 may pick another token where two
    logits are within rounding: every emitted token must be within twice the logits' bound of the
    plain arg-max at its position (teacher-forced on the emitted tokens)."""
    if dtype == "float32":
        assert tokens == plain.greedy(model, prompt, len(tokens))
        return
    lg = plain.logits(model, list(prompt) + list(tokens[:-1]))[len(prompt) - 1:]
    scale = lg.abs().max().item()
    for step, (row, tok) in enumerate(zip(lg, tokens)):
        gap = row.max().item() - row[tok].item()
        assert gap <= 2 * helpers.TOL[dtype] * scale, (step, tok, gap, scale)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point(engines, plains, folders, dtype):
    for tag in ("A_sharp", "B", "D"):
        cfg = CONFIGS[tag][0]
        eng = engines(tag, dtype)
        lens = (5, 9, 13) if tag == "A_sharp" else (1, 7, 16, 31)
        prompts = tiny_models.random_prompts(cfg, lens, seed=60)
        steps = list(eng.generate(prompts, 12))
        assert len(steps) == 12 and all(len(s) == len(prompts) for s in steps)
        got = [[s[b] for s in steps] for b in range(len(prompts))]
        assert got == eng.generate_all(prompts, 12)
        for p, g in zip(prompts, got):
            check_tokens_against_plain(plains[tag], p, g, dtype)
        # the outputs are not one repeated token: an engine stuck after its first step would show
        assert max(len(set(plain.greedy(plains[tag], p, 12))) for p in prompts) >= 6


def test_sampling_through_the_entry_point(engines, plains):
    """Temperature 0.8 with a fixed seed on configuration B: same draws as the plain rule."""
    tag = "B"
    cfg = CONFIGS[tag][0]
    eng = engines(tag, "float32")
    prompts = tiny_models.random_prompts(cfg, (1, 7, 16, 31), seed=61)
    got = eng.generate_all(prompts, 12, temperature=0.8, top_k=0, seed=1234)
    again = eng.generate_all(prompts, 12, temperature=0.8, top_k=0, seed=1234)
    assert got == again

    def plain_draws(prompt, stream, n, temperature, top_k, seed):
        ids, out = list(prompt), []
        for step in range(n):
            row = plain.logits(plains[tag], ids)[-1]
            out.append(plain.sample_token(row, temperature, top_k, seed, stream, step))
            ids.append(out[-1])
        return out
    for b, p in enumerate(prompts):
        assert got[b] == plain_draws(p, b, 12, 0.8, 0, 1234), b
    # draws depend on the request's index in its call, not on batch mates: request 2 alone is
    # stream 0 of its call and draws what the plain rule draws for stream 0
    alone = eng.generate_all([prompts[2]], 12, temperature=0.8, seed=1234)
    assert alone[0] == plain_draws(prompts[2], 0, 12, 0.8, 0, 1234)
    assert alone[0] != got[2], "streams 0 and 2 should not draw alike over 12 tokens"
    topk = eng.generate_all(prompts, 6, temperature=1.5, top_k=3, seed=7)
    for b, p in enumerate(prompts):
        ids = list(p)
        for step, tok in enumerate(topk[b]):
            row = plain.logits(plains[tag], ids)[-1]
            assert tok in torch.topk(row, 3).indices.tolist()
            assert tok == plain.sample_token(row, 1.5, 3, 7, b, step)
            ids.append(tok)


def test_stop_tokens_and_early_end(engines, plains):
    """A stop token that first appears inside the captured decode steps ends its sequence there,
    while its batch mates go on exactly as they would alone; a budget of 2 ends another one."""
    tag = "A_sharp"
    cfg = CONFIGS[tag][0]
    eng = engines(tag, "float32")
    prompts = tiny_models.random_prompts(cfg, (5, 9, 13), seed=60)
    free = [plain.greedy(plains[tag], p, 10) for p in prompts]
    # a token of request 1 that first appears at step 2 or later and that requests 0 and 2 never emit
    stop, first = next((tok, i) for i, tok in enumerate(free[1])
                       if i >= 2 and free[1].index(tok) == i and tok not in free[0] and tok not in free[2])
    out = eng.generate_all(prompts, [10, 10, 2], stop_token_ids=[stop])
    assert out[0] == free[0]                           # untouched by its mates' ends
    assert out[1] == free[1][:first + 1]               # the stop token is kept as the last one
    assert out[2] == free[2][:2]                       # its budget
    steps = list(eng.generate(prompts, 10, stop_token_ids=[stop]))
    cols = [[s[b] for s in steps] for b in range(3)]
    assert cols[0] == free[0] and cols[2] == free[2]
    assert cols[1][:first + 1] == free[1][:first + 1] and all(t == -1 for t in cols[1][first + 1:])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_step_larger_than_one_pass_is_cut_into_pieces(folders, plains, dtype):
    """More tokens than one pass takes: sequences are cut inside, later pieces read the cache
    the earlier ones left, and the wanted rows come back in the caller's order."""
    from enginekernel_b200 import Engine
    tag = "C"
    cfg = CONFIGS[tag][0]
    eng = Engine(folders[tag], dtype, max_tokens=2048, max_batch=4, max_step_tokens=50)
    seqs = tiny_models.random_prompts(cfg, [120, 7, 77], seed=91)
    slots = [eng.open_sequence() for _ in seqs]
    wants = [[0, 119, 60, 49, 50], [6], list(range(77))[::-1]]
    logits = eng.step([(s, q, w) for s, q, w in zip(slots, seqs, wants)]).cpu()
    r = 0
    for q, w in zip(seqs, wants):
        ref = plain.logits(plains[tag], q)
        for place in w:
            err = (logits[r] - ref[place]).abs().max().item() / ref.abs().max().item()
            assert err <= helpers.TOL[dtype], (len(q), place, err)
            r += 1
    assert r == logits.shape[0]
    for s in slots:
        eng.close_sequence(s)


def test_more_than_64_sequences_decode_together(folders, plains):
    """A decode step wider than the small-batch kernels take (bfloat16)."""
    from enginekernel_b200 import Engine
    tag = "B"
    cfg = CONFIGS[tag][0]
    eng = Engine(folders[tag], "bfloat16", max_tokens=64 * 80, max_batch=80)
    seqs = tiny_models.random_prompts(cfg, [3 + (i % 5) for i in range(70)], seed=17)
    got = helpers.batch_then_steps(eng, seqs, [len(s) - 2 for s in seqs])
    for i in (0, 1, 33, 69):
        assert helpers.rel_err(got[i], plain.logits(plains[tag], seqs[i])) <= helpers.TOL["bfloat16"]


def test_a_prompt_step_of_more_sequences_than_the_tile_table_takes(folders, plains):
    """1,100 short prompts in one step: the tcgen05 prompt attention takes 1,024 sequences a step, so
    this step runs on the mma.sync kernel instead of being refused (head size 64, bfloat16)."""
    from enginekernel_b200 import Engine
    tag = "E"
    cfg = CONFIGS[tag][0]
    n = 1100
    eng = Engine(folders[tag], "bfloat16", max_tokens=64 * n, max_batch=n)
    seqs = tiny_models.random_prompts(cfg, [2 + (i % 4) for i in range(n)], seed=23)
    slots = [eng.open_sequence() for _ in seqs]
    logits = eng.step([(slot, s, [len(s) - 1]) for slot, s in zip(slots, seqs)]).cpu()
    for slot in slots:
        eng.close_sequence(slot)
    eng.runner.check_kernels()
    for i in (0, 511, 1023, 1024, 1099):
        want = plain.logits(plains[tag], seqs[i])[-1:]
        assert helpers.rel_err(logits[i:i + 1], want) <= helpers.TOL["bfloat16"], i


def test_sizes_the_tensor_core_path_cannot_address_still_work(tmp_path):
    """A width that is a multiple of 4 but not of 8: bfloat16 falls back to the library product
    instead of refusing or computing wrong."""
    from enginekernel_b200 import Engine
    cfg = dict(tiny_models.TINY_A, hidden_size=68, intermediate_size=100, vocab_size=131)
    folder = helpers.make_folder(tmp_path / "odd", cfg, 5)
    model = helpers.plain_model(folder)
    ids = tiny_models.random_prompts(cfg, [40], seed=2)[0]
    want = plain.logits(model, ids)
    for dtype in ("float32", "bfloat16"):
        eng = Engine(folder, dtype, max_tokens=256, max_batch=2)
        assert helpers.rel_err(helpers.whole(eng, ids), want) <= helpers.TOL[dtype]
        assert helpers.rel_err(helpers.tail_one_by_one(eng, ids, 8), want) <= helpers.TOL[dtype]


@pytest.mark.parametrize("tag", ["A", "C", "D", "E"])
def test_norms_moved_into_the_products_change_rounding_only(engines, plains, tag):
    """With few rows the residual add and the norm ride on the products around them; the logits
    must agree with the norm kernel's, and with the plain implementation, as closely as before."""
    from enginekernel_b200.ops import linear, kernels
    cfg = CONFIGS[tag][0]
    ids = tiny_models.random_prompts(cfg, [min(90, cfg["max_position_embeddings"])], seed=77)[0]
    want = plain.logits(plains[tag], ids)
    eng = engines(tag, "bfloat16")
    calls = []
    real = kernels.gemm_tc_bf16

    def spy(*a, **kw):
        calls.append((kw.get("row_scale") is not None, kw.get("residual") is not None))
        return real(*a, **kw)
    got = {}
    limit = linear.DEFER_NORM_ROWS
    try:
        kernels.gemm_tc_bf16 = spy
        for rows in (limit, 0):
            linear.DEFER_NORM_ROWS = rows
            calls.clear()
            got[rows] = helpers.tail_one_by_one(eng, ids, 32)
            took = any(s or r for s, r in calls)
            assert took == (rows > 0), "the deferred form runs exactly when it is allowed"
    finally:
        linear.DEFER_NORM_ROWS = limit
        kernels.gemm_tc_bf16 = real
    assert helpers.rel_err(got[limit], want) <= helpers.TOL["bfloat16"]
    assert helpers.rel_err(got[0], want) <= helpers.TOL["bfloat16"]
    assert helpers.rel_err(got[limit], got[0]) <= helpers.TOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_decode(tmp_path, dtype):
    """4,200 cached tokens for one sequence: 66 cache pages, so the decode attention cuts them
    over as many blocks as the device allows a cluster (16 where it can); a second, shorter
    sequence decodes beside it and ends earlier."""
    from enginekernel_b200 import Engine
    cfg = dict(tiny_models.TINY_E, max_position_embeddings=8192, num_hidden_layers=2)
    folder = helpers.make_folder(tmp_path, cfg, 5)
    model = helpers.plain_model(folder)
    eng = Engine(folder, dtype, max_tokens=2 * 4352, max_batch=2)
    seqs = tiny_models.random_prompts(cfg, [4208, 1300], seed=9)
    got = helpers.batch_then_steps(eng, seqs, [4200, 1296])
    for s, g in zip(seqs, got):
        want = plain.logits(model, s)
        tail = slice(len(s) - 12, len(s))
        err = helpers.rel_err(g[tail], want[tail])
        assert err <= helpers.TOL[dtype], (dtype, len(s), err)


@pytest.mark.parametrize("shape", [
    dict(num_attention_heads=3, num_key_value_heads=1, head_dim=256, hidden_size=72),     # one KV head
    dict(num_attention_heads=10, num_key_value_heads=2, head_dim=96, hidden_size=160),    # groups of 5
    dict(num_attention_heads=2, num_key_value_heads=2, head_dim=128, hidden_size=48),     # no grouping
    dict(num_attention_heads=40, num_key_value_heads=2, head_dim=64, hidden_size=200),    # groups of 20
])
def test_unusual_head_shapes(tmp_path, shape):
    """Head sizes and groupings at the edges of what the kernels take, whole and one by one."""
    from enginekernel_b200 import Engine
    cfg = dict(tiny_models.TINY_C, **shape)
    folder = helpers.make_folder(tmp_path, cfg, 6)
    model = helpers.plain_model(folder)
    eng = Engine(folder, "bfloat16", max_tokens=1024, max_batch=2)
    ids = tiny_models.random_prompts(cfg, [150], seed=13)[0]
    want = plain.logits(model, ids)
    assert helpers.rel_err(helpers.whole(eng, ids), want) <= helpers.TOL["bfloat16"]
    assert helpers.rel_err(helpers.tail_one_by_one(eng, ids, 20), want) <= helpers.TOL["bfloat16"]


def poison_free_pages(engine, value=1e4):
    """Fill every cache page no sequence holds with large finite keys and values of both signs:
    enough to move any logit whose attention read them, too small to overflow."""
    for g in engine.cache.groups:
        if g.page_group is None:
            continue
        free = torch.tensor(sorted(g.page_group.pool._free), dtype=torch.long, device=g.pages.device)
        if free.numel() == 0:
            continue
        shape = g.pages[:, :, free].shape
        signs = torch.where(torch.arange(shape[-1], device=g.pages.device) % 2 == 0, value, -value)
        g.pages[:, :, free] = signs.to(g.pages.dtype).expand(shape)
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["B", "D", "E"])
def test_stale_pages_change_nothing(folders, plains, tag, dtype):
    """Pages handed to a sequence hold whatever their last owner (or nobody) left there.  With every
    free page filled with +-1e4 before each batch, logits and generated tokens are what they were:
    no kernel reads a key beyond a sequence's length, not even with a weight of almost nothing."""
    from enginekernel_b200 import Engine
    cfg = CONFIGS[tag][0]
    eng = Engine(folders[tag], dtype, max_tokens=12 * 64, max_batch=3)
    seqs = tiny_models.random_prompts(cfg, [70, 5, 130], seed=71)
    wants = [plain.logits(plains[tag], s) for s in seqs]
    for round_ in range(2):                       # the second round reuses pages the first one wrote
        poison_free_pages(eng)
        got = helpers.batch_then_steps(eng, seqs, [64, 3, 120])
        for s, g, w in zip(seqs, got, wants):
            err = helpers.rel_err(g, w)
            assert err <= helpers.TOL[dtype], (tag, dtype, round_, len(s), err)
    prompts = [s[:n] for s, n in zip(seqs, (63, 5, 100))]
    poison_free_pages(eng)
    for p, toks in zip(prompts, eng.generate_all(prompts, 20)):
        check_tokens_against_plain(plains[tag], p, toks, dtype)
    assert eng.cache.free_tokens() == eng.cache.num_pages * 64
