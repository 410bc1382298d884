"""Single-process CPU checks of the model-level machinery: sequence
micro-batching, the fused loss path, cached prefill/decode, scoring,
checkpoint round trips."""
import json
import os

import pytest
import torch


def _cfg(**kw):
    from megalodon_b200.config import ModelConf
    base = dict(num_layers=2, model_dim=64, num_heads=2, z_dim=32, value_dim=128, ffn_hidden_dim=128,
                cema_ndim=4, chunk_size=16, vocab_size=96, swiglu=True, norm_num_groups=8)
    base.update(kw)
    return ModelConf(**base)


def _build(cfg, seed=0, dtype="fp32"):
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.utils import set_random_seed
    set_random_seed(seed)
    return build_model(cfg, dtype, False, True)


def _grads(model):
    model.finish_backward()
    return torch.cat([p.grad.flatten() for p in model.parameters() if p.grad is not None])


@pytest.mark.parametrize("ckpt", [False, True])
def test_sequence_microbatching_matches_full(ckpt):
    from megalodon_b200.modules.losses import cross_entropy
    cfg = _cfg(layerwise_ckpt=ckpt)
    toks = torch.randint(0, 96, (2, 65), generator=torch.Generator().manual_seed(3))
    x, y = toks[:, :-1], toks[:, 1:]
    outs = []
    for k in (None, 1, 2):
        model = _build(cfg)
        model.materialize_fp32_grads = True
        model.seq_microbatch_chunks = k
        model._wrapped.seq_microbatch_chunks = k
        pred, _ = model(x)
        loss = cross_entropy(pred, y).mean()
        loss.backward()
        outs.append((pred.detach(), loss.item(), _grads(model)))
    for pred, loss, g in outs[1:]:
        assert torch.allclose(pred, outs[0][0], atol=1e-4, rtol=1e-4)
        assert abs(loss - outs[0][1]) < 1e-5
        assert torch.allclose(g, outs[0][2], atol=1e-5, rtol=1e-3), (g - outs[0][2]).abs().max()


def test_fused_loss_path_matches_logits_path():
    from megalodon_b200.modules.losses import cross_entropy
    cfg = _cfg()
    toks = torch.randint(0, 96, (2, 49), generator=torch.Generator().manual_seed(4))
    x, y = toks[:, :-1], toks[:, 1:]
    res = []
    for fused, k in ((False, None), (True, None), (True, 1)):
        model = _build(cfg)
        model.materialize_fp32_grads = True
        model._wrapped.seq_microbatch_chunks = k
        if fused:
            tok_loss, _ = model(x, targets=y)
        else:
            pred, _ = model(x)
            tok_loss = cross_entropy(pred, y)
        tok_loss.mean().backward()
        res.append((tok_loss.detach(), _grads(model)))
    for tl, g in res[1:]:
        assert torch.allclose(tl, res[0][0], atol=1e-5, rtol=1e-5)
        assert torch.allclose(g, res[0][1], atol=1e-6, rtol=1e-4)


def test_cached_prefill_and_decode_match_full_forward():
    from megalodon_b200.models.mega import Mega
    from megalodon_b200.utils import init_cache, set_random_seed
    cfg = _cfg(efficient_attn="fused")
    set_random_seed(0)
    model = Mega(cfg).eval()
    toks = torch.randint(0, 96, (2, 16 * 3 + 5), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        # reference: feed whole chunks at once, then the 5-token tail, all with cache
        full_a, cache = model(toks[:, :48], cache=init_cache(2, model, torch.float32))
        # incremental: 2 chunks, 1 chunk, then token by token
        cache2 = init_cache(2, model, torch.float32)
        p1, cache2 = model(toks[:, :32], cache=cache2)
        p2, cache2 = model(toks[:, 32:48], cache=cache2)
        assert torch.allclose(torch.cat([p1, p2], 1), full_a, atol=1e-4, rtol=1e-4)
        tail_ref, _ = model(toks[:, 48:], cache=cache)
        steps = []
        for t in range(48, 53):
            o, cache2 = model(toks[:, t:t + 1], cache=cache2)
            steps.append(o)
        assert torch.allclose(torch.cat(steps, 1), tail_ref, atol=1e-4, rtol=1e-4)
        # no-cache forward over whole chunks equals the cached one
        nocache, _ = model(toks[:, :48])
        assert torch.allclose(nocache, full_a, atol=1e-4, rtol=1e-4)


def test_inference_scoring_and_generation():
    from megalodon_b200.models.mega import Mega
    from megalodon_b200.inference import inference
    from megalodon_b200.generation import generate, sample_top_k, sample_top_p
    from megalodon_b200.utils import set_random_seed
    cfg = _cfg()
    set_random_seed(0)
    model = Mega(cfg).eval()
    toks = torch.randint(0, 96, (2, 16 * 9 + 4), generator=torch.Generator().manual_seed(6))
    x, y = toks[:, :-1], toks[:, 1:].clone()
    y[1, -7:] = -100
    nll = inference(model, x, y, "fp32")
    assert nll.shape == x.shape and torch.isfinite(nll).all()
    assert (nll[1, -7:] == 0).all()
    # short sequences (no truncation kicks in) agree with a plain forward
    with torch.no_grad():
        pred, _ = model(x[:, :64])
        ref = torch.nn.functional.cross_entropy(pred.flatten(0, 1), y[:, :64].flatten(), reduction="none")
    assert torch.allclose(inference(model, x[:, :64], y[:, :64], "fp32").flatten(), ref, atol=1e-4)

    class Tok:
        bos_id, eos_id, pad_id, n_words = 1, 2, 0, 96

        def encode(self, s, bos, eos):
            return ([self.bos_id] if bos else []) + [3 + (ord(ch) % 90) for ch in s]

    out = generate(model, "fp32", Tok(), prompt=["hello world, this is a prompt", "short"], max_gen_len=6)
    assert len(out) == 2 and all(len(o) == 6 for o in out)
    out2 = generate(model, "fp32", Tok(), prompt=["hello world, this is a prompt", "short"], max_gen_len=6)
    assert out == out2          # greedy decoding is deterministic
    # the fixed-shape decode session (what CUDA models use by default) produces the same tokens
    out3 = generate(model, "fp32", Tok(), prompt=["hello world, this is a prompt", "short"], max_gen_len=6,
                    use_decode_session=True)
    assert out3 == out
    long_a = generate(model, "fp32", Tok(), prompt=["ab"], max_gen_len=40)
    long_b = generate(model, "fp32", Tok(), prompt=["ab"], max_gen_len=40, use_decode_session=True)
    assert long_a == long_b     # 40 tokens cross several chunk boundaries
    probs = torch.softmax(torch.randn(3, 50), -1)
    assert sample_top_k(probs.clone(), 5).shape == (3, 1)
    assert sample_top_p(probs.clone(), 0.8).shape == (3, 1)


def test_checkpoint_roundtrips(tmp_path):
    from megalodon_b200 import reloading
    from megalodon_b200.config import OptimConf
    from megalodon_b200.models.mega import Mega
    from megalodon_b200.optim import build_optimizer
    cfg = _cfg(share_emb=True)
    model = _build(cfg, seed=1)
    opt, sched = build_optimizer(model, OptimConf(lr=1e-2, warmup=1), 10, "fp32")
    toks = torch.randint(0, 96, (2, 33), generator=torch.Generator().manual_seed(7))
    x, y = toks[:, :-1], toks[:, 1:]

    def step(m, o, s):
        loss = m(x, targets=y)[0].mean()
        loss.backward()
        m.clip_grad_norm_(1.0)
        o.step(); s.step(); o.zero_grad()
        return loss.item()

    step(model, opt, sched)
    # key list of the consolidated format
    sd = model.state_dict()
    expected = {"embed.weight", "rope.freqs", "output.output.weight", "output.final_norm.weight",
                "output.final_norm.bias", "output.final_norm.prior_count", "output.final_norm.prior_mean",
                "output.final_norm.prior_logv"}
    for i in range(2):
        pre = f"layers.{i}."
        expected |= {pre + k for k in (
            "mega.timenorm.prior_count", "mega.timenorm.prior_mean", "mega.timenorm.prior_logv",
            "mega.timenorm.weight", "mega.timenorm.bias", "mega.cema.alpha", "mega.cema.delta",
            "mega.cema.theta", "mega.cema.gamma", "mega.cema.omega", "mega.rmsnorm.weight",
            "mega.wv.weight", "mega.wv.bias", "mega.wz.weight", "mega.wz.bias", "mega.wr.weight",
            "mega.wr.bias", "mega.wh1.weight", "mega.wh1.bias", "mega.wh2.weight", "mega.gamma", "mega.beta",
            "nffn.norm.weight", "nffn.norm.bias", "nffn.fc1.weight", "nffn.fc2.weight", "nffn.fc3.weight")}
    assert set(sd.keys()) == expected, set(sd.keys()) ^ expected
    assert sd["layers.0.mega.wz.weight"].shape == (32, 64)
    assert sd["layers.0.mega.gamma"].shape == (2, 32)

    # sharded save -> resume gives the same next loss as continuing
    reloading.save_sharded(model, opt, sched, 1, str(tmp_path / "sharded"), cfg)
    cont = step(model, opt, sched)
    model2 = _build(cfg, seed=99)
    opt2, sched2 = build_optimizer(model2, OptimConf(lr=1e-2, warmup=1), 10, "fp32")
    assert reloading.load_sharded(model2, opt2, sched2, str(tmp_path / "sharded")) == 1
    assert abs(step(model2, opt2, sched2) - cont) < 1e-6

    # offline consolidation of the sharded checkpoint, then load into a plain model
    reloading.consolidate(str(tmp_path / "sharded"), str(tmp_path / "cons"), dtype="fp32")
    assert (tmp_path / "cons" / "consolidated.pth").exists()
    cc = json.load(open(tmp_path / "cons" / "consolidate_config.json"))
    assert cc == {"model_parallel_size": 1, "dtype": "fp32"}
    state = torch.load(tmp_path / "cons" / "consolidated.pth")
    plain = Mega(cfg)
    missing, unexpected = plain.load_state_dict(state, strict=False)
    assert not unexpected and not missing, (missing, unexpected)

    # online consolidated save equals the model's own state dict
    reloading.save_consolidated(model2, str(tmp_path / "cons2"), cfg, dtype="fp32")
    st2 = torch.load(tmp_path / "cons2" / "consolidated.pth")
    for k, v in model2.state_dict().items():
        assert torch.equal(st2[k], v), k
    rc = reloading.reload_config(tmp_path / "cons2")
    assert not rc.is_fsdp and rc.mp_world_size == 1 and rc.dtype == "fp32"


def test_checkpointed_model_saves_and_reloads_under_the_plain_key_names(tmp_path):
    """A model trained with activation checkpointing writes the same key names as one without
    (fairscale's checkpoint_wrapper, which the reference uses, does not rename keys); reloading builds
    the evaluation model without checkpointing, every tensor equals the file's, and a file that
    lacks a parameter is refused instead of leaving uninitialised weights."""
    from megalodon_b200 import reloading
    from megalodon_b200.config import TokenizerConf
    from megalodon_b200.models.mega import Mega
    cfg = _cfg(layerwise_ckpt=True, ckpt_layers=1)
    model = _build(cfg, seed=3)
    plain_keys = set(_build(_cfg(), seed=3).state_dict().keys())
    assert set(model.state_dict().keys()) == plain_keys
    reloading.save_consolidated(model, str(tmp_path / "cons"), cfg, dtype="fp32")
    state = torch.load(tmp_path / "cons" / "consolidated.pth")
    assert set(state.keys()) == plain_keys

    import json
    saved = json.load(open(tmp_path / "cons" / "config.json"))
    assert saved["model"]["layerwise_ckpt"] is True
    known = set(type(cfg).__dataclass_fields__)
    mcfg = type(cfg)(**{k: v for k, v in saved["model"].items() if k in known})
    mcfg.init_mode = "none"
    for wrapped_too in (False, True):              # the file loads into either kind of model
        mcfg.layerwise_ckpt, mcfg.ckpt_layers = wrapped_too, None
        ev = Mega(mcfg)
        reloading.load_state_dict(ev, dict(state), strict=False)
        got = ev.state_dict()
        for k, v in state.items():
            assert torch.equal(got[k], v), k
    # same outputs as the trained model
    toks = torch.randint(0, 96, (2, 32), generator=torch.Generator().manual_seed(5))
    ev.eval(); model.eval()
    with torch.no_grad():
        assert torch.allclose(ev(toks)[0], model(toks)[0], atol=1e-5)
    broken = {k: v for k, v in state.items() if k != "layers.1.mega.wz.weight"}
    with pytest.raises(RuntimeError, match="no value for 1 parameter"):
        reloading.load_state_dict(Mega(mcfg), broken, strict=False)


def test_decode_session_matches_cache_path():
    """The fixed-shape decode state reproduces the regular cache path token for token, from a prefilled
    cache and from an empty one, across a chunk boundary."""
    from megalodon_b200.config import ModelConf
    from megalodon_b200.decoding import DecodeSession
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.utils import init_cache, set_random_seed
    cfg = ModelConf(num_layers=2, model_dim=64, num_heads=2, z_dim=32, value_dim=64, ffn_hidden_dim=64,
                    cema_ndim=4, chunk_size=8, vocab_size=50, swiglu=True, norm_num_groups=8)
    set_random_seed(0)
    model = build_model(cfg, "fp32", device=torch.device("cpu"))
    model.eval()
    inner = model._wrapped
    B = 2
    prompt = torch.randint(0, 50, (B, 11))
    with torch.no_grad():
        cache = init_cache(B, inner, torch.float32, device=torch.device("cpu"))
        _, cache = model(prompt[:, :8], cache=cache)
        logits, cache = model(prompt[:, 8:], cache=cache)
        sess = DecodeSession(model, B, torch.float32, use_graph=False)
        sess.load_cache(cache)
        t_ref = t_ses = logits[:, -1].argmax(-1)
        for _ in range(14):
            ref, cache = model(t_ref.view(B, 1), cache=cache)
            got = sess.step(t_ses)
            assert torch.allclose(ref[:, -1], got, atol=1e-5, rtol=1e-5)
            t_ref, t_ses = ref[:, -1].argmax(-1), got.argmax(-1)
        cache = init_cache(B, inner, torch.float32, device=torch.device("cpu"))
        sess = DecodeSession(model, B, torch.float32, use_graph=False)
        tok = torch.randint(0, 50, (B,))
        for _ in range(10):
            ref, cache = model(tok.view(B, 1), cache=cache)
            got = sess.step(tok)
            assert torch.allclose(ref[:, -1], got, atol=1e-5, rtol=1e-5)
            tok = ref[:, -1].argmax(-1)
    model.train()        # the module tree must stay acyclic after forwards
    model.eval()


def test_reference_import_paths_resolve_to_this_package():
    """`megalodon.*` module paths of the reference are the same module objects as `megalodon_b200.*`."""
    import megalodon.model.mega as a
    import megalodon_b200.model.mega as b
    assert a is b
    from megalodon.distributed import initialize_model_parallel, get_chunk_parallel_world_size  # noqa: F401
    from megalodon.model.mega import build_model as bm
    from megalodon.modules import FusedLayerNorm, FusedRMSNorm, MovingAverageGatedAttention, TimestepNorm  # noqa: F401
    from megalodon.modules.fused_ops import (ema_hidden, ema_parameters, fftconv, fused_fftconv_bwd,  # noqa: F401
                                             fused_fftconv_fwd, memory_efficient_dropout, swift_efficient_attention,
                                             swift_efficient_attention_bwd, swift_efficient_attention_fwd)
    from megalodon.optim import build_optimizer, rescale_grads  # noqa: F401
    from megalodon.utils import clip_grad_norm_, init_cache, set_random_seed  # noqa: F401
    from megalodon.reloading import reload_model  # noqa: F401
    from megalodon.inference import inference  # noqa: F401
    from megalodon.generation import generate  # noqa: F401
    import megalodon_b200.models.mega as c
    assert bm is c.build_model
    x = torch.randn(2, 3, 9)
    k = torch.randn(3, 9)
    g = torch.randn(2, 3, 9)
    dx, dk = fused_fftconv_bwd(g, x, k)
    assert dx.shape == x.shape and dk.shape == k.shape
    q = torch.randn(1, 5, 2, 4)
    v = torch.randn(1, 5, 2, 6)
    dq, dk2, dv = swift_efficient_attention_bwd(torch.randn(1, 5, 2, 6), q, q.clone(), v)
    assert dq.shape == q.shape and dv.shape == v.shape


def test_partial_checkpointing_gives_the_same_gradients():
    """Checkpointing only the first k blocks (ModelConf.ckpt_layers) changes memory, not numbers."""
    from megalodon_b200.config import ModelConf
    from megalodon_b200.models.mega import build_model
    from megalodon_b200.utils import set_random_seed
    base = dict(num_layers=3, model_dim=64, num_heads=2, z_dim=32, value_dim=64, ffn_hidden_dim=64, cema_ndim=4,
                chunk_size=8, vocab_size=50, swiglu=True, norm_num_groups=8)
    toks = torch.randint(0, 50, (2, 17))
    x, y = toks[:, :-1], toks[:, 1:]
    grads = []
    for kw in (dict(layerwise_ckpt=False), dict(layerwise_ckpt=True, ckpt_layers=1), dict(layerwise_ckpt=True)):
        set_random_seed(0)
        model = build_model(ModelConf(**base, **kw), "fp32", device=torch.device("cpu"))
        model._wrapped.seq_microbatch_chunks = 1
        from megalodon_b200.parallel.checkpoint import CheckpointWrapper
        n_wrapped = sum(isinstance(m, CheckpointWrapper) for m in model.modules())
        assert n_wrapped == (0 if not kw["layerwise_ckpt"] else kw.get("ckpt_layers", 3))
        loss = model(x, targets=y)[0].mean()
        loss.backward()
        model.finish_backward()
        grads.append(torch.cat([p._grad_shard.float().reshape(-1) for p in model.parameters()]))
    assert torch.allclose(grads[0], grads[1], atol=1e-6, rtol=1e-5)
    assert torch.allclose(grads[0], grads[2], atol=1e-6, rtol=1e-5)
