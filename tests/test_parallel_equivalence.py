"""N-rank result == 1-rank result for forward, loss, gradient norm and one
AdamW step, over data / chunk / model parallel layouts on CPU (gloo)."""
import pytest
import torch

from dist_utils import run_ranks


def _tiny_cfg(**kw):
    from megalodon_b200.config import ModelConf
    base = dict(num_layers=2, model_dim=64, num_heads=2, z_dim=32, value_dim=128, ffn_hidden_dim=128,
                cema_ndim=4, chunk_size=16, vocab_size=96, swiglu=True, norm_num_groups=8)
    base.update(kw)
    return ModelConf(**base)


def _train_steps(rank, world, mp, cp, cfg_kw, shard_cp, steps, dtype):
    import torch.distributed as dist
    from megalodon_b200.parallel import initialize_model_parallel, get_data_parallel_rank, \
        get_data_parallel_world_size
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.optim import build_optimizer
    from megalodon_b200.config import OptimConf
    from megalodon_b200.modules.losses import cross_entropy
    from megalodon_b200.utils import clip_grad_norm_, set_random_seed
    if world > 1 or mp * cp > 1:
        initialize_model_parallel(mp, cp)
    set_random_seed(1234)
    cfg = _tiny_cfg(**cfg_kw)
    model = build_model(cfg, dtype, False, True, shard_over_chunk_group=shard_cp)
    opt, sched = build_optimizer(model, OptimConf(lr=1e-2, warmup=1, weight_decay=0.1), 10, dtype)
    g = torch.Generator().manual_seed(7)
    dp = get_data_parallel_world_size()
    all_toks = torch.randint(0, cfg.vocab_size, (4, 65), generator=g)
    per = 4 // dp
    toks = all_toks[get_data_parallel_rank() * per:(get_data_parallel_rank() + 1) * per]
    x, y = toks[:, :-1], toks[:, 1:]
    out = []
    for _ in range(steps):
        pred, _ = model(x)
        loss = cross_entropy(pred, y).mean()
        loss.backward()
        model.grad_all_reduce()
        norm = clip_grad_norm_(model, 1.0)
        opt.step(); sched.step(); opt.zero_grad()
        lsum = loss.detach().clone()
        if dp > 1:
            from megalodon_b200.parallel import get_data_parallel_group
            dist.all_reduce(lsum, group=get_data_parallel_group())
            lsum /= dp
        out.append((lsum.item(), float(norm)))
    sd = model.state_dict()
    return out, {k: v.float() for k, v in sd.items()}


def _gather_mp(states, key, mp):
    """Concatenate model-parallel slices of `key` (first mp ranks = one replica)."""
    parts = [states[r][key] for r in range(mp)]
    if parts[0].dim() == 0 or ".rmsnorm." in key or ".nffn.norm." in key:
        return parts[0]
    col = ("wv.weight", "wz.weight", "wr.weight", "wh1.weight", "fc1.weight", "fc3.weight")
    row = ("wh2.weight", "fc2.weight", "embed.weight", "output.output.weight")
    if key.endswith(col):
        return torch.cat(parts, 0)
    if key.endswith(row):
        return torch.cat(parts, 1)
    if key.endswith(("gamma", "beta")) and parts[0].dim() == 2 and ".mega." in key and "cema" not in key:
        return torch.cat(parts, 1)
    return torch.cat(parts, 0)


LAYOUTS = [
    # world, mp, cp, shard_over_cp
    (2, 1, 1, False),     # dp = 2
    (2, 1, 2, False),     # cp = 2, replicated + grad_all_reduce
    (2, 1, 2, True),      # cp = 2, sharded over the chunk group
    (2, 2, 1, False),     # mp = 2
    (4, 1, 4, False),     # cp = 4
    (4, 2, 2, False),     # mp = 2 x cp = 2
    (4, 1, 2, True),      # dp = 2 x cp = 2 sharded over both
]


@pytest.fixture(scope="module")
def baseline():
    res = run_ranks(_train_steps, 1, 1, 1, {}, False, 2, "fp32")
    return res[0]


@pytest.mark.parametrize("world,mp,cp,shard_cp", LAYOUTS)
def test_layout_matches_single_rank(baseline, world, mp, cp, shard_cp):
    base_curve, base_state = baseline
    res = run_ranks(_train_steps, world, mp, cp, {}, shard_cp, 2, "fp32")
    curve = res[0][0]
    for (l0, n0), (l1, n1) in zip(base_curve, curve):
        assert abs(l0 - l1) < 2e-4 * max(1.0, abs(l0)), (base_curve, curve)
        assert abs(n0 - n1) < 2e-3 * max(1.0, abs(n0)), (base_curve, curve)
    states = [r[1] for r in res]
    for key, ref in base_state.items():
        if key == "rope.freqs":
            continue
        got = _gather_mp(states, key, mp) if mp > 1 else states[0][key]
        assert got.shape == ref.shape, (key, got.shape, ref.shape)
        assert torch.allclose(got, ref, atol=2e-4, rtol=2e-3), (key, (got - ref).abs().max())


def test_checkpointing_and_bf16_run():
    res = run_ranks(_train_steps, 2, 1, 2, {"layerwise_ckpt": True}, False, 2, "fp32")
    base = run_ranks(_train_steps, 1, 1, 1, {}, False, 2, "fp32")
    for (l0, n0), (l1, n1) in zip(base[0][0], res[0][0]):
        assert abs(l0 - l1) < 2e-4 * max(1.0, abs(l0))
        assert abs(n0 - n1) < 2e-3 * max(1.0, abs(n0))
    res16 = run_ranks(_train_steps, 2, 1, 1, {}, False, 2, "bf16")
    assert all(torch.isfinite(torch.tensor(l)) for l, _ in res16[0][0])
    assert abs(res16[0][0][0][0] - base[0][0][0][0]) < 0.1


def _decode_case(rank, world, mp):
    """Prefill through the regular cache path, then decode through the fixed-shape session."""
    from megalodon_b200.decoding import DecodeSession
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.utils import init_cache, set_random_seed
    if world > 1:
        initialize_model_parallel(mp, 1)
    set_random_seed(1234)
    cfg = _tiny_cfg()
    model = build_model(cfg, "fp32", False, False)
    model.eval()
    inner = model._wrapped
    B = 2
    prompt = torch.randint(0, cfg.vocab_size, (B, 16 + 5), generator=torch.Generator().manual_seed(3))
    outs = []
    with torch.no_grad():
        cache = init_cache(B, inner, torch.float32, device=torch.device("cpu"))
        _, cache = model(prompt[:, :16], cache=cache)
        logits, cache = model(prompt[:, 16:], cache=cache)
        sess = DecodeSession(model, B, torch.float32, use_graph=False)
        sess.load_cache(cache)
        tok = logits[:, -1].argmax(-1)
        for _ in range(14):                      # positions 5 .. 18 of the chunk: crosses the boundary at 16
            lg = sess.step(tok)
            outs.append(lg.clone())
            tok = lg.argmax(-1)
    return torch.stack(outs)


def test_decode_session_under_tensor_parallelism_matches_single_rank():
    single = run_ranks(_decode_case, 1, 1)[0]
    for got in run_ranks(_decode_case, 2, 2):
        assert torch.allclose(got, single, atol=2e-4, rtol=2e-4), (got - single).abs().max()


def _prefill_decode_case(rank, world, cp):
    """Chunk-parallel prefill that emits a cache, then replicated decode through the cache path."""
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.utils import init_cache, set_random_seed
    if world > 1:
        initialize_model_parallel(1, cp)
    set_random_seed(1234)
    cfg = _tiny_cfg()
    model = build_model(cfg, "fp32", False, False, shard_over_chunk_group=cp > 1)
    model.eval()
    inner = model._wrapped
    B, c = 2, cfg.chunk_size
    prompt = torch.randint(0, cfg.vocab_size, (B, 4 * c), generator=torch.Generator().manual_seed(5))
    outs = []
    with torch.no_grad():
        if cp > 1:
            inner.seq_microbatch_chunks = 1          # two pieces per rank: exercises the carry as well
            logits, cache = model(prompt, prefill=True)
        else:
            cache = init_cache(B, inner, torch.float32, device=torch.device("cpu"))
            for s in range(0, 4 * c, 2 * c):
                full, cache = model(prompt[:, s:s + 2 * c], cache=cache)
            logits = full[:, -1]
        outs.append(logits.clone())
        tok = logits.argmax(-1)
        for _ in range(6):
            lg, cache = model(tok.view(B, 1), cache=cache)
            outs.append(lg[:, -1].clone())
            tok = lg[:, -1].argmax(-1)
    return torch.stack(outs)


def test_chunk_parallel_prefill_hands_its_state_to_decode():
    single = run_ranks(_prefill_decode_case, 1, 1)[0]
    for got in run_ranks(_prefill_decode_case, 2, 2):
        assert torch.allclose(got, single, atol=2e-4, rtol=2e-4), (got - single).abs().max()


def _cache_case(rank, world, mp):
    """Cache after prefilling one and a half chunks through the regular cache path."""
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.utils import init_cache, set_random_seed
    if world > 1:
        initialize_model_parallel(mp, 1)
    set_random_seed(1234)
    cfg = _tiny_cfg()
    model = build_model(cfg, "fp32", False, False)
    model.eval()
    B, c = 2, cfg.chunk_size
    prompt = torch.randint(0, cfg.vocab_size, (B, c + c // 2), generator=torch.Generator().manual_seed(9))
    with torch.no_grad():
        cache = init_cache(B, model._wrapped, torch.float32, device=torch.device("cpu"))
        _, cache = model(prompt[:, :c], cache=cache)
        _, cache = model(prompt[:, c:], cache=cache)
    return cache


def test_more_tensor_parallel_ranks_than_heads():
    """4 ranks on a 2-head model: each head's value columns are split over two ranks, its shared q/k
    projection is replicated on them.  Decoding must match the single-rank model."""
    single = run_ranks(_decode_case, 1, 1)[0]
    for got in run_ranks(_decode_case, 4, 4):
        assert torch.allclose(got, single, atol=2e-4, rtol=2e-4), (got - single).abs().max()


@pytest.mark.parametrize("mp", [2, 4])
def test_reshard_cache_matches_a_tensor_parallel_cache(mp):
    from megalodon_b200.utils import reshard_cache
    full = run_ranks(_cache_case, 1, 1)[0]
    per_rank = run_ranks(_cache_case, mp, mp)
    for r, (layers, out_norm) in enumerate(per_rank):
        exp_layers, exp_out = reshard_cache(full, r, mp)
        for (kv, norm, hx), (ekv, enorm, ehx) in zip(layers, exp_layers):
            assert kv[2] == ekv[2]
            for a, b in list(zip(kv[:2], ekv[:2])) + list(zip(norm, enorm)):
                assert a.shape == b.shape and torch.allclose(a.float(), b.float(), atol=1e-4, rtol=1e-4)
            assert torch.allclose(torch.view_as_real(hx), torch.view_as_real(ehx), atol=1e-4, rtol=1e-4)
        for a, b in zip(out_norm, exp_out):
            assert torch.allclose(a.float(), b.float(), atol=1e-4, rtol=1e-4)


def _state_case(rank, world, mp):
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.parallel import initialize_model_parallel
    from megalodon_b200.utils import set_random_seed
    if world > 1:
        initialize_model_parallel(mp, 1)
    set_random_seed(77)
    model = build_model(_tiny_cfg(rescale_nffn=True), "fp32", False, False)
    # make the zero-initialised parameters distinguishable
    with torch.no_grad():
        g = torch.Generator().manual_seed(5)
        sd = model.state_dict()
    return {k: v.clone() for k, v in sd.items()}


@pytest.mark.parametrize("mp", [2, 4])
def test_full_state_dict_slices_to_any_tensor_parallel_size(mp):
    """`shard_state_dict_for_model_parallel` of the single-rank model equals, key by key, what a
    model built on `mp` tensor-parallel ranks from the same seed holds (4 ranks on 2 heads included)."""
    from megalodon_b200.reloading import shard_state_dict_for_model_parallel
    full = run_ranks(_state_case, 1, 1)[0]
    per_rank = run_ranks(_state_case, mp, mp)
    for r, sd in enumerate(per_rank):
        want = shard_state_dict_for_model_parallel(full, 2, r, mp)
        assert set(want) == set(sd), set(want) ^ set(sd)
        for k in sd:
            assert want[k].shape == sd[k].shape, (k, want[k].shape, sd[k].shape)
            assert torch.equal(want[k], sd[k]), k


def _switch_case(rank, world):
    """Chunk-parallel prefill on `world` ranks, then tensor-parallel decode on the same ranks with the
    weights and the state handed over inside the process (what `infer_bench.py --phase both` does)."""
    from megalodon_b200.decoding import DecodeSession
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.parallel import (destroy_model_parallel, get_model_parallel_rank,
                                         initialize_model_parallel)
    from megalodon_b200.reloading import shard_state_dict_for_model_parallel
    from megalodon_b200.utils import expand_cache, init_cache, reshard_cache, set_random_seed
    cfg = _tiny_cfg()
    B, c = 1, cfg.chunk_size
    prompt = torch.randint(0, cfg.vocab_size, (B, 4 * c), generator=torch.Generator().manual_seed(11))
    outs = []
    with torch.no_grad():
        if world == 1:
            set_random_seed(1234)
            model = build_model(cfg, "fp32", False, False)
            model.eval()
            cache = init_cache(B, model._wrapped, torch.float32, device=torch.device("cpu"))
            for s in range(0, 4 * c, 2 * c):
                full, cache = model(prompt[:, s:s + 2 * c], cache=cache)
            logits = full[:, -1]
            decoder, state = model, cache
        else:
            initialize_model_parallel(1, world)
            set_random_seed(1234)
            model = build_model(cfg, "fp32", False, False, shard_over_chunk_group=True)
            model.eval()
            logits, cache = model(prompt, prefill=True)
            full_sd = {k: v.clone() for k, v in model.gathered_state_dict().items()}
            destroy_model_parallel()
            initialize_model_parallel(world, 1)
            set_random_seed(999)                               # the decoder's own initialisation must not matter
            decoder = build_model(cfg, "fp32", False, False)
            decoder.eval()
            r = get_model_parallel_rank()
            decoder.load_state_dict(shard_state_dict_for_model_parallel(full_sd, cfg.num_heads, r, world), strict=False)
            state = reshard_cache(cache, r, world)
        outs.append(logits.clone())
        sess = DecodeSession(decoder, 2, torch.float32, use_graph=False)
        sess.load_cache(expand_cache(state, 2))
        tok = logits.argmax(-1).expand(2)
        for _ in range(6):
            lg = sess.step(tok)
            outs.append(lg[:1].clone())
            tok = lg.argmax(-1)
    return torch.cat(outs)


@pytest.mark.parametrize("world", [2, 4])
def test_prefill_layout_hands_over_to_decode_layout(world):
    single = run_ranks(_switch_case, 1)[0]
    for got in run_ranks(_switch_case, world):
        assert torch.allclose(got, single, atol=3e-4, rtol=3e-4), (got - single).abs().max()
