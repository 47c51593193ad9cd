"""The Tufevik design through the engine against the plain implementation (``tests/plain/tufevik_plain.py``): both mixers
alone and together, whole prompts, decoding through pages and states, portions down to two tokens, mixed batches with
pages and slots that are used again, other sizes, both precisions, greedy generation through ``LLMEngine``; and the
kernels of its mechanisms alone, with inputs made so that a lost key, a window that is one token off or a state that
is not carried shows."""
import json
import random
import tempfile
from pathlib import Path
from types import SimpleNamespace

import pytest
import torch

import helpers
from plain import tufevik_plain as plain

pytestmark = pytest.mark.gpu


def moe(experts=5, top=2, ff=40):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def dense(ff=88):
    return {"kind": "dense", "ff": ff}


def memory(heads=3, dim=16, vdim=24, cap=8.0, mlp="default"):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap},
            "mlp": dense() if mlp == "default" else mlp}


def side_by_side(heads=4, kv_heads=2, dim=16, vdim=24, conv=4, scale=None, rot_dims=8, base=10000.0, factor=4.0,
                 original=64, inner=48, state=6, dt_rank=5, taps=3, left_scale=0.6, right_scale=1.4, mlp="default",
                 fast=8.0, slow=1.0):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
            "scale": scale if scale is not None else 1.5 / dim ** 0.5,
            "rot": {"base": base, "dims": rot_dims,
                    "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}}
    right = {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": taps}
    return {"type": "parallel", "mlp": moe() if mlp == "default" else mlp,
            "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def model(layers, width=64, vocab=211, embed_scale=0.5, eps=1e-5, positions=1024):
    return {"architecture": "Tufevik", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "max_position_embeddings": positions}


CONFIGS = {
    "memory_only": model([memory(), memory(heads=2, dim=32, vdim=32, mlp=None), memory(heads=4, dim=8, vdim=16, mlp=moe())]),
    "side_by_side_only": model([side_by_side(), side_by_side(heads=6, kv_heads=3, dim=8, vdim=8, mlp=None, taps=4, conv=2),
                                side_by_side(heads=2, kv_heads=1, dim=32, vdim=16, rot_dims=32, mlp=dense())]),
    "both_kinds": model([side_by_side(), memory(), memory(heads=2, dim=32, vdim=16, mlp=moe(experts=3, top=3)),
                         side_by_side(heads=8, kv_heads=2, dim=16, vdim=16, inner=96, state=16, dt_rank=4, mlp=dense()),
                         memory(mlp=None)], width=80),
    # values that many models make equal or one: one head, one key/value head per query head, one tap (a convolution
    # that only scales), every dimension rotated, a stretch factor of one, scores and branches unscaled, one state a
    # channel, a step-size rank of one, one expert chosen and one expert in all, an embedding constant of one
    "equal_or_one": model([side_by_side(heads=1, kv_heads=1, dim=32, vdim=32, conv=1, scale=1.0, rot_dims=32, factor=1.0,
                                        inner=32, state=1, dt_rank=1, taps=1, left_scale=1.0, right_scale=1.0,
                                        mlp=moe(experts=4, top=1)),
                           memory(heads=1, dim=32, vdim=32, mlp=moe(experts=1, top=1, ff=64)),
                           side_by_side(heads=3, kv_heads=3, dim=16, vdim=16, rot_dims=2, mlp=None)],
                          width=64, embed_scale=1.0),
    # sizes that no vector load or few-rows product takes; more states than a lane keeps; more taps than most; a
    # rotated part that is a few values of a head; a head of the memory wider than 32 rows and a value of one column
    "odd_sizes": model([side_by_side(heads=9, kv_heads=3, dim=20, vdim=12, conv=5, rot_dims=6, inner=37, state=23, dt_rank=3,
                                     taps=2, mlp=moe(experts=7, top=4, ff=18)),
                        memory(heads=5, dim=12, vdim=28, mlp=None),
                        memory(heads=1, dim=72, vdim=1, cap=2.5, mlp=dense(ff=50)),
                        side_by_side(heads=5, kv_heads=1, dim=12, vdim=28, conv=3, rot_dims=12, inner=70, state=3, dt_rank=9,
                                     taps=6, base=77.0, factor=2.5, original=40, fast=4.0, slow=0.5, mlp=dense(ff=34))],
                       width=102, vocab=333),
}
# float32: the recurrences pass rounding on from token to token through exponentials of differences, and a memory's
# read-out divides by a sum that may nearly cancel and norms what is left (a head of one value most of all): the
# largest row errors measured are 1.1e-4 of the logits' size, hundreds of tokens in.  A lost key, a window that is one
# token off or a state that is not carried moves a row by a hundredth and more.
RMS_LIMIT = {"float32": 3.0e-4, "bfloat16": 1.0e-1}
_MODELS: dict = {}


def folder_of(name: str):
    if name not in _MODELS:
        holder = tempfile.TemporaryDirectory(prefix=f"tufevik_{name}_")
        plain.write_model(holder.name, CONFIGS[name], seed=41 + len(_MODELS))
        _MODELS[name] = (holder, Path(holder.name), plain.load_folder(holder.name))
    return _MODELS[name][1]


def reference(name: str, tokens):
    folder_of(name)
    config, weights = _MODELS[name][2]
    return plain.forward_full(config, weights, tokens).to(torch.float32)


def replay(name: str, dtype: str, steps, max_tokens: int, page: int = 16, max_requests: int = 4):
    from llm_serving_engine_b200.engine.trace_replay import replay as run

    with tempfile.TemporaryDirectory(prefix="tufevik_out_") as out:
        run(folder_of(name), dtype, out, max_tokens, [json.dumps(step) for step in steps], block_size=page,
            max_requests=max_requests)
        return helpers.collect(steps, Path(out))


def compare(name, dtype, requests, got, what):
    """Row error over logit size, per position.  float32: every row within the limit.  bfloat16: a router's choice
    between two almost equal logits may fall the other way than in the plain implementation, which moves that row by
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


@pytest.mark.parametrize("name", ["both_kinds", "odd_sizes", "equal_or_one"])
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
    from llm_serving_engine_b200.kernels import ops

    seen = []

    def after_layer(position, stream):
        """A layer's last output is still pending with its norm (the next layer's norm adds it): add it to a copy."""
        residual = stream.residual.clone()
        if stream.delta is not None:
            ops.tanh_norm(residual, stream.delta, stream.delta_norm.triple, None, None)
        seen.append(residual.cpu())

    engine_model.layer_hook = after_layer
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
    """Decoding reads the pages, windows and states that the prompt step left (single tokens are replayed from a
    captured graph); a prompt of one token and of fewer tokens than a convolution has taps are among them."""
    requests = some_requests(name, [40, 9, 3, 25], seed=6)
    got = replay(name, dtype, helpers.trace_tail_decode(requests, tail=24), helpers.max_tokens_for(requests))
    compare(name, dtype, requests, got, "tail decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["both_kinds", "odd_sizes"])
def test_portions_of_changing_size(name, dtype):
    """Portions shorter than the convolutions' windows, portions that end on a page's and a chunk's border, one
    token at a time between longer ones."""
    requests = some_requests(name, [150, 33], seed=7)
    for sizes in ((7, 2, 13, 3, 2, 31, 5, 16, 2, 64, 17), (2,), (16, 16, 1, 15, 17), (1, 2, 3, 1, 1, 64, 63)):
        got = replay(name, dtype, helpers.trace_portions(requests, sizes), helpers.max_tokens_for(requests))
        compare(name, dtype, requests, got, f"portions {sizes}")


def test_a_long_prompt_is_scanned_in_chunks_and_in_portions_alike():
    """A prompt long enough for the chunked form of the memory's scan (chunks side by side, a carry between them),
    whole and in portions that cut chunks anywhere."""
    for name in ("both_kinds", "memory_only"):
        requests = some_requests(name, [413], seed=13)
        whole = replay(name, "float32", helpers.trace_whole(requests), 448)
        compare(name, "float32", requests, whole, "long whole")
        cut = replay(name, "float32", helpers.trace_portions(requests, (130, 1, 199, 65, 2)), 448)
        compare(name, "float32", requests, cut, "long in portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page", [16, 8])
def test_mixed_batches_reuse_pages_and_slots(dtype, page):
    """Nine requests through four slots and a pool sized for the live ones only: a page's old rows must not be read,
    and a slot's memory, scan state, maximum and windows must start from zero for the request that takes it next."""
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
    """600 single tokens after a short prompt: the keys pass the borders of tiles, chunks and many pages, and the
    recurrent states are carried six hundred times."""
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
def _step(lengths, first_positions=None, slots=None):
    """The step's tensors that the kernels read, for requests of ``lengths`` rows laid one after the other."""
    first_positions = first_positions or [0] * len(lengths)
    slots = slots if slots is not None else list(range(len(lengths)))
    seg, pos, start = [], [], [0]
    for index, (count, first) in enumerate(zip(lengths, first_positions)):
        seg += [index] * count
        pos += list(range(first, first + count))
        start.append(start[-1] + count)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device="cuda")
    return SimpleNamespace(segment_of_token=as_int(seg), positions=as_int(pos), segment_start=as_int(start),
                           segment_first_position=as_int(first_positions), segment_state_slot=as_int(slots))


def _cuts(total, sizes):
    """(first row, rows) of the portions of ``sizes``, repeated until ``total`` rows are spent."""
    out, at, index = [], 0, 0
    while at < total:
        size = min(sizes[index % len(sizes)], total - at)
        out.append((at, size))
        at, index = at + size, index + 1
    return out


@pytest.mark.parametrize("width", [64, 102])
def test_tanh_norm_adds_and_norms(width):
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(4)
    rows = 37
    residual, delta = torch.randn(rows, width) * 2, torch.randn(rows, width) * 3
    after = (torch.tensor([0.7]), torch.rand(width) + 0.5, torch.randn(width) * 0.2)
    before = (torch.tensor([1.3]), torch.rand(width) + 0.5, torch.randn(width) * 0.2)
    norm = lambda x, triple: torch.tanh(triple[0].double() * x.double()) * triple[1].double() + triple[2].double()
    want_residual = residual.double() + norm(delta, after)
    want_out = norm(want_residual, before)
    cuda = lambda triple: tuple(t.cuda() for t in triple)
    for stacked in (False, True):
        for out_dtype, limit in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
            r = residual.clone().cuda()
            d = torch.stack([delta * 0.25, delta * 0.75]).cuda().contiguous() if stacked else delta.cuda()
            out = torch.empty(rows, width, dtype=out_dtype, device="cuda")
            ops.tanh_norm(r, d, cuda(after), cuda(before), out)
            assert float((r.cpu().double() - want_residual).abs().max()) <= 2e-6 * float(want_residual.abs().max())
            assert float((out.float().cpu().double() - want_out).abs().max()) <= limit * float(want_out.abs().max())
    # some rows only (the rows whose logits are asked for), no delta
    r = residual.clone().cuda()
    pick = torch.tensor([36, 0, 5], dtype=torch.int32, device="cuda")
    out = torch.empty(3, width, dtype=torch.float32, device="cuda")
    ops.tanh_norm(r, None, None, cuda(before), out, rows=pick)
    assert float((out.cpu().double() - norm(residual, before)[pick.cpu().long()]).abs().max()) <= 2e-6 * 2
    assert torch.equal(r.cpu(), residual)


@pytest.mark.parametrize("taps", [1, 2, 4, 6])
def test_a_short_convolution_sees_its_taps_and_no_more(taps):
    """One row of ones among zeros: the rows after it show the taps from the last to the first, the row after those
    shows nothing.  The marked row lies before, at and after the cuts between steps, in portions down to one row,
    for two requests in one step whose windows lie in slots of their own."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(5)
    channels, total, offset = 37, 40, 3
    weight = (torch.randn(channels, taps) + 2.0)
    bias = torch.randn(channels)
    for marked in (0, 1, 6, 7, 8, 20):
        u = torch.zeros(2, total, offset + channels + 2)
        u[0, marked, offset:offset + channels] = 1.0
        u[1] = torch.randn(total, offset + channels + 2)        # a neighbour whose rows must not leak
        want = [plain.causal_conv(u[r, :, offset:offset + channels].double(), weight.double(), bias.double()) for r in (0, 1)]
        for row in range(total):        # what the plain convolution says about the marked row
            j = row - marked
            expected = weight[:, taps - 1 - j].double() + bias.double() if 0 <= j < taps else bias.double()
            assert torch.allclose(want[0][row], expected)
        for sizes in ((total,), (7, 1, 1, 2, 13), (2,), (1,)):
            state = torch.zeros(5, max(taps - 1, 0), channels, device="cuda")
            state[1], state[4] = 7.0, -7.0      # other requests' windows
            got = [[], []]
            for first, count in _cuts(total, sizes):
                step = _step([count, count], [first, first], slots=[3, 0])
                proj = torch.cat([u[0, first:first + count], u[1, first:first + count]]).cuda().contiguous()
                out = torch.empty(2 * count, channels, device="cuda")
                ops.short_conv_act(proj, offset, weight.cuda(), bias.cuda(), state, step, out, "none")
                if taps > 1:
                    ops.short_conv_state(proj, offset, channels, taps, state, step)
                got[0].append(out[:count].cpu())
                got[1].append(out[count:].cpu())
            for r in (0, 1):
                assert float((torch.cat(got[r]).double() - want[r]).abs().max()) <= 1e-5, (marked, sizes, r)
            if taps > 1:
                assert float((state[1] - 7.0).abs().max()) == 0.0 and float((state[4] + 7.0).abs().max()) == 0.0
                assert torch.allclose(state[3].cpu(), u[0, total - taps + 1:, offset:offset + channels])


@pytest.mark.parametrize("heads,dim,vdim", [(3, 16, 24), (1, 72, 1), (2, 128, 128), (4, 8, 33)])
def test_matrix_memory_gates_scan_and_read_out(heads, dim, vdim):
    """Gates from wide-open to shut (pre-activations beyond the cap on both sides), so that the running maximum moves,
    stays and falls; whole, in chunks side by side, and in portions down to one row, the state carried between them."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(6)
    total, cap, eps = 203, 6.0, 1e-5
    qk, val = heads * dim, heads * vdim
    width = 2 * qk + 2 * val + 2 * heads
    proj = torch.randn(2, total, width)
    proj[:, :, -2 * heads:] *= 5.0                      # the gates' pre-activations
    proj[0, :40, -2 * heads:-heads] = -9.0              # a request that starts with its input gate shut ...
    proj[0, 40:44, -2 * heads:-heads] = 11.0            # ... then wide open
    i_bias, f_bias = torch.randn(heads), torch.randn(heads) + 1.0
    weight = torch.rand(val) + 0.5
    want = []
    for r in (0, 1):
        p = proj[r].double()
        q = p[:, :qk].view(total, heads, dim) * dim ** -0.5
        k = p[:, qk:2 * qk].view(total, heads, dim)
        v = p[:, 2 * qk:2 * qk + val].view(total, heads, vdim)
        gate = torch.sigmoid(p[:, 2 * qk + val:2 * qk + 2 * val])
        i = plain.capped(p[:, -2 * heads:-heads] + i_bias.double(), cap)
        f = torch.nn.functional.logsigmoid(plain.capped(p[:, -heads:] + f_bias.double(), cap))
        read = plain.rms(plain.mlstm_recurrence(q, k, v, i, f), eps).reshape(total, val)
        want.append(read * weight.double() * gate)
    for sizes, chunked in (((total,), True), ((total,), False), ((64, 1, 2, 65, 1, 1, 3), None), ((2,), None)):
        memory = torch.zeros(4, heads, dim, vdim + 1, device="cuda")
        maximum = torch.zeros(4, heads, device="cuda")
        memory[1], maximum[1] = 3.0, 2.0       # another request's state
        got = [[], []]
        for first, count in _cuts(total, sizes):
            step = _step([count, count], [first, first], slots=[2, 0])
            rows = torch.cat([proj[0, first:first + count], proj[1, first:first + count]]).cuda().contiguous()
            keep, take, floor = ops.mlstm_gates(rows, width - 2 * heads, width - heads, i_bias.cuda(), f_bias.cuda(), cap,
                                                maximum, step.segment_start, step.segment_state_slot, heads)
            read = torch.empty(2 * count, heads * (vdim + 1), device="cuda")
            ops.gated_linear_attention_scan(rows, 0, qk, 2 * qk, keep, take, dim ** -0.5, memory, step.segment_start,
                                            step.segment_state_slot, read, heads, dim, vdim, chunked=chunked)
            out = torch.empty(2 * count, val, device="cuda")
            ops.mlstm_readout(read, floor, rows, 2 * qk + val, weight.cuda(), eps, out, heads, vdim, step.segment_of_token)
            got[0].append(out[:count].cpu())
            got[1].append(out[count:].cpu())
        for r in (0, 1):
            error = (torch.cat(got[r]).double() - want[r]).abs()
            assert float(error.max()) <= 3e-4 * float(want[r].abs().max()), (sizes, chunked, r, int(error.max(1).values.argmax()))
        assert float((memory[1] - 3.0).abs().max()) == 0.0 and float((maximum[1] - 2.0).abs().max()) == 0.0


@pytest.mark.parametrize("channels,states,rank", [(48, 6, 5), (37, 23, 3), (128, 16, 8), (32, 1, 1), (20, 100, 2)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_selective_scan_and_its_step_sizes(channels, states, rank, dtype):
    """Step sizes from tiny to large (slow and fast forgetting), whole and in portions down to one row, two requests
    in a step with slots of their own; the bfloat16 form takes bfloat16 inputs and keeps float32 states."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(7)
    total, z_off = 150, 5
    x = torch.randn(2, total, channels).to(dtype).float()
    proj = torch.randn(2, total, z_off + channels)                       # z after some other columns
    low = torch.randn(2, total, rank + 2 * states + 3)
    dt_weight, dt_bias = torch.randn(channels, rank) * 1.5, torch.randn(channels) - 2.0
    a_log, skip = torch.log(torch.rand(channels, states) * 4 + 0.2), torch.rand(channels) + 0.5
    want, want_dt = [], []
    for r in (0, 1):
        dt = torch.nn.functional.softplus(low[r, :, :rank].double() @ dt_weight.double().t() + dt_bias.double())
        y = plain.selective_scan(x[r].double(), dt, -torch.exp(a_log.double()), low[r, :, rank:rank + states].double(),
                                 low[r, :, rank + states:rank + 2 * states].double(), skip.double())
        want.append(y * torch.nn.functional.silu(proj[r, :, z_off:].double()) * 0.75)
        want_dt.append(dt)
    for sizes in ((total,), (17, 1, 2, 16, 1, 33), (2,), (1,)):
        state = torch.zeros(3, channels, states, device="cuda")
        state[1] = 5.0
        got = [[], []]
        for first, count in _cuts(total, sizes):
            step = _step([count, count], [first, first], slots=[2, 0])
            pick = lambda t: torch.cat([t[0, first:first + count], t[1, first:first + count]]).cuda().contiguous()
            rows_low = pick(low)
            dt = ops.ssm_step_sizes(rows_low, dt_weight.t().contiguous().cuda(), dt_bias.cuda())
            assert float((dt[:count].cpu().double() - want_dt[0][first:first + count]).abs().max()) <= 1e-5 * float(want_dt[0].max())
            wide = torch.zeros(2 * count, channels + 4, dtype=dtype, device="cuda")      # the output is a column range
            ops.selective_scan(pick(x).to(dtype), dt, pick(proj), z_off, rows_low, rank, rank + states, a_log.cuda(), skip.cuda(),
                               state, step, wide[:, 4:], 0.75)
            assert float(wide[:, :4].float().abs().max()) == 0.0
            got[0].append(wide[:count, 4:].float().cpu())
            got[1].append(wide[count:, 4:].float().cpu())
        limit = 2e-5 if dtype == torch.float32 else 6e-3
        for r in (0, 1):
            error = (torch.cat(got[r]).double() - want[r]).abs()
            assert float(error.max()) <= limit * float(want[r].abs().max()), (sizes, r, int(error.max(1).values.argmax()))
        assert float((state[1] - 5.0).abs().max()) == 0.0


def _left_branch(proj, offset, conv, q_norm, k_norm, rot, cuts, sizes, scale, eps, page, dtype=torch.float32, first=0):
    """The attention side's kernels over one request whose rows come in the portions ``cuts``: convolutions, norms,
    rotation and page writes, then the paged attention, then the heads' gates.  Pages lie scattered in a pool whose
    other rows hold NaN."""
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.parts.latent_attention import rotary_frequencies

    n_q, n_kv, dk, dv = sizes
    channels, taps, total = (n_q + n_kv) * dk + n_kv * dv, conv.shape[1], proj.shape[0]
    pages = -(-(first + total) // page)
    order = torch.randperm(pages + 4, generator=torch.Generator().manual_seed(total + page))[:pages].to(torch.int32)
    keys = torch.full((pages + 4, n_kv, page, dk), float("nan"), dtype=dtype, device="cuda")
    values = torch.full((pages + 4, n_kv, page, dv), float("nan"), dtype=dtype, device="cuda")
    window = torch.zeros(2, max(taps - 1, 0), channels, device="cuda")
    freq, factor = rotary_frequencies(rot)
    out = []
    for at, count in cuts:
        step = _step([count], [first + at], slots=[1])
        rows = proj[at:at + count].cuda().contiguous()
        places = torch.arange(first + at, first + at + count)
        slots = (order[places // page].long() * page + places % page).to(torch.int32).cuda()
        q = torch.empty(count, n_q, dk, dtype=dtype, device="cuda")
        gate = torch.empty(count, n_q, device="cuda")
        ops.conv_qk_norm_rope(rows, offset, offset + channels, conv.cuda(), window, q_norm.cuda(), k_norm.cuda(), eps,
                              freq.to(torch.float64).contiguous().cuda(), factor, step, slots, q, keys, values, gate,
                              n_q, n_kv, dk, dv)
        if taps > 1:
            ops.short_conv_state(rows, offset, channels, taps, window, step)
        attended = torch.empty(count, n_q, dv, dtype=dtype, device="cuda")
        ops.attention_scored(q, keys, values, attended, order.view(1, -1).cuda(), step.segment_of_token, step.positions, scale,
                             segment_start=step.segment_start, segment_first_position=step.segment_first_position)
        gated = torch.empty(count, n_q * dv, dtype=dtype, device="cuda")
        ops.head_gate_scale(attended, gate, gated, 0.5, step.segment_of_token)
        out.append(gated.float().cpu())
    return torch.cat(out)


def _plain_left_branch(proj, offset, conv, q_norm, k_norm, rot, sizes, scale, eps):
    n_q, n_kv, dk, dv = sizes
    total, a, b = proj.shape[0], n_q * dk, (n_q + n_kv) * dk
    u = proj[:, offset:].double()
    q = plain.causal_conv(u[:, :a], conv[:a].double())
    k = plain.causal_conv(u[:, a:b], conv[a:b].double())
    v = plain.causal_conv(u[:, b:b + n_kv * dv], conv[b:].double())
    q, k = plain.rms(q, eps) * q_norm.double(), plain.rms(k, eps) * k_norm.double()
    cos, sin = plain.rotary_table(rot, total)
    q = plain.rotate_half(q.view(total, n_q, dk), cos, sin, int(rot["dims"]))
    k = plain.rotate_half(k.view(total, n_kv, dk), cos, sin, int(rot["dims"]))
    out = plain.causal_softmax_attention(q, k, v.view(total, n_kv, dv), scale)
    gate = torch.sigmoid(u[:, b + n_kv * dv:b + n_kv * dv + n_q])
    return (out * gate[:, :, None] * 0.5).reshape(total, n_q * dv), q


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_convolved_attention_finds_one_far_key_at_every_border(dtype):
    """One key among hundreds is made to stand out for one head of the last row (behind the convolution: the marked
    row's input is solved for, and the marked values lie in the part of a head that is not rotated); it sits at, just
    before and just after the borders of pages and of key tiles and chunks, as the first key and as the last row's
    neighbour.  The rows come as one prompt, as a prompt and a single token (keys split over blocks and merged), and
    in portions of two."""
    torch.manual_seed(8)
    sizes = n_q, n_kv, dk, dv = 4, 2, 24, 40
    offset, page, context, eps, scale, taps = 2, 16, 300, 1e-5, 1.2, 3
    rot = {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}
    channels = (n_q + n_kv) * dk + n_kv * dv
    conv = torch.randn(channels, taps) * 0.3
    conv[:, -1] = 1.0 + torch.rand(channels)
    q_norm, k_norm = torch.rand(n_q * dk) + 0.5, torch.rand(n_kv * dk) + 0.5
    for special in (0, 1, 15, 16, 17, 31, 32, 255, 256, 257, 297, 298):
        proj = (torch.randn(context, offset + channels + n_q) * 0.5).to(dtype).float()
        u = proj[:, offset:]
        q_conv = plain.causal_conv(u[:, :n_q * dk].double(), conv[:n_q * dk].double())[context - 1].view(n_q, dk)
        k_cols = slice(n_q * dk + 8, n_q * dk + dk)                    # key/value head 0, the values that are not rotated
        k_conv = plain.causal_conv(u[:, k_cols].double(), conv[k_cols].double())[special]
        target = 6.0 * q_conv[1, 8:] * q_norm[dk + 8:2 * dk].double() / k_norm[8:dk].double()      # k after its norm is a multiple of q after its norm
        u[special, k_cols] += ((target - k_conv) / conv[k_cols, -1].double()).float()
        proj = proj.to(dtype).float()
        want, _ = _plain_left_branch(proj, offset, conv, q_norm, k_norm, rot, sizes, scale, eps)
        unmarked = proj.clone()
        unmarked[special, offset + k_cols.start:offset + k_cols.stop] = 0.0
        other, _ = _plain_left_branch(unmarked, offset, conv, q_norm, k_norm, rot, sizes, scale, eps)
        if special < context - taps:       # the marked key carries the last row: a kernel that lost it would show
            assert float((other[-1] - want[-1]).abs().max()) > 0.05, special
        for cuts in ([(0, context)], [(0, context - 1), (context - 1, 1)], _cuts(context, (2,)) if special in (16, 257) else None):
            if cuts is None:
                continue
            got = _left_branch(proj, offset, conv, q_norm, k_norm, rot, cuts, sizes, scale, eps, page, dtype)
            limit = 3e-5 if dtype == torch.float32 else 4e-2
            error = (got.double() - want).abs()
            assert float(error.max()) <= limit * max(1.0, float(want.abs().max())), (special, len(cuts), int(error.max(1).values.argmax()))


def test_rotation_far_from_the_start_and_stretched_frequencies():
    """Rows at positions beyond thirty thousand (angles of thousands of turns, taken in float32 from float64
    frequencies): the rotated queries against the plain table, for frequencies that are stretched, not stretched and in
    between, all of a head rotated and a few of its values; cosine and sine carry the stretch's factor."""
    from llm_serving_engine_b200.kernels import ops
    from llm_serving_engine_b200.parts.latent_attention import rotary_frequencies

    torch.manual_seed(9)
    n_q, n_kv, dk, dv, eps, count = 3, 1, 32, 8, 1e-6, 6
    channels = (n_q + n_kv) * dk + n_kv * dv
    for dims, scaling in ((32, {"factor": 8.0, "original": 512, "fast": 32.0, "slow": 1.0}), (6, {"factor": 1.0, "original": 64, "fast": 2.0, "slow": 1.0}),
                          (16, {"factor": 2.5, "original": 4096, "fast": 4.0, "slow": 0.25}), (0, None)):
        rot = {"base": 50000.0, "dims": dims, "scaling": scaling}
        freq, factor = rotary_frequencies(rot) if dims else (torch.zeros(0, dtype=torch.float64), 1.0)
        for first in (0, 31000):
            proj = torch.randn(count, channels)
            step = _step([count], [first], slots=[0])
            keys = torch.zeros(3000, n_kv, 16, dk, device="cuda") if first == 0 else keys
            values = torch.zeros(3000, n_kv, 16, dv, device="cuda") if first == 0 else values
            slots = torch.arange(first, first + count, dtype=torch.int32, device="cuda")
            q = torch.empty(count, n_q, dk, device="cuda")
            ops.conv_qk_norm_rope(proj.cuda(), 0, 0, torch.ones(channels, 1, device="cuda"), torch.zeros(1, 0, channels, device="cuda"),
                                  torch.ones(n_q * dk, device="cuda"), torch.ones(n_kv * dk, device="cuda"), eps,
                                  freq.to(torch.float64).contiguous().cuda(), factor, step, slots, q, keys, values, None, n_q, n_kv, dk, dv)
            want = plain.rms(proj[:, :n_q * dk].double(), eps).view(count, n_q, dk)
            want_k = plain.rms(proj[:, n_q * dk:(n_q + n_kv) * dk].double(), eps).view(count, n_kv, dk)
            if dims:
                cos, sin = plain.rotary_table(rot, count, first)
                want, want_k = plain.rotate_half(want, cos, sin, dims), plain.rotate_half(want_k, cos, sin, dims)
            assert float((q.cpu().double() - want).abs().max()) <= 2e-5, (dims, first)
            written = keys.view(-1, n_kv, 16, dk)[first // 16:(first + count) // 16 + 1].transpose(1, 2).reshape(-1, n_kv, dk)
            assert float((written[first % 16:first % 16 + count].cpu().double() - want_k).abs().max()) <= 2e-5, (dims, first)


@pytest.mark.parametrize("experts,top", [(5, 2), (1, 1), (7, 7), (16, 4), (4, 1)])
def test_router_weights_are_the_softmax_over_the_chosen_logits(experts, top):
    """The largest logits (bias added) are chosen; their weights add up to one and are not the shares that a softmax
    over all experts would give them."""
    from llm_serving_engine_b200.kernels import ops

    torch.manual_seed(10)
    rows = 50
    logits, bias = torch.randn(rows, experts + 3) * 2, torch.randn(experts) * 2
    chosen = torch.empty(rows, top, dtype=torch.int32, device="cuda")
    weights, _, _ = ops.moe_route(logits.cuda(), None, experts, 0, top, chosen=chosen, logit_bias=bias.cuda(), over_chosen=True)
    full = logits[:, :experts].double() + bias.double()
    values, picked = torch.topk(full, top, dim=-1)
    want = torch.zeros(rows, experts, dtype=torch.float64).scatter(1, picked, torch.softmax(values, dim=-1))
    assert torch.equal(chosen.cpu().long().sort(dim=1).values, picked.sort(dim=1).values)
    assert float((weights.cpu().double() - want).abs().max()) <= 2e-6
    assert float((weights.sum(1).cpu() - 1.0).abs().max()) <= 1e-5
    if top < experts:
        over_all = torch.softmax(full, dim=-1) * (want > 0)
        assert float((over_all - want).abs().max()) > 0.01


def test_command_line_generates_from_a_model_folder_and_from_the_stand_in():
    """``bin/llmserve generate`` on a folder of the design (the class comes from config.json): the greedy tokens are the
    plain implementation's; and on the random stand-in of the design."""
    import os
    import subprocess
    import sys

    root = str(Path(__file__).resolve().parent.parent)
    env = dict(os.environ, PYTHONPATH=root)
    name, prompt, count = "both_kinds", [5, 17, 3, 150, 99, 42, 7], 8
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "llmserve"), "generate", "--model", str(folder_of(name)),
                          "--dtype", "float32", "--prompt-ids", " ".join(map(str, prompt)), "--max-new-tokens", str(count)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    tokens = json.loads(out.stdout.strip().splitlines()[-1])["output_ids"]
    assert len(tokens) == count
    logits = reference(name, prompt + tokens)
    for index, token in enumerate(tokens):
        row = logits[len(prompt) + index - 1]
        top = torch.topk(row, 2).values
        if float(top[0] - top[1]) < 1e-3 * float(row.abs().max()):
            break
        assert int(row.argmax()) == token, f"token {index}"
    out = subprocess.run([sys.executable, os.path.join(root, "bin", "llmserve"), "generate", "--random", "tufevik",
                          "--prompt-ids", "5 17 3 250 99", "--max-new-tokens", "6"],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stderr
    assert len(json.loads(out.stdout.strip().splitlines()[-1])["output_ids"]) == 6
