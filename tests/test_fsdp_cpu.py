"""Single-process checks of the FSDP wrapper's gradient bookkeeping (CPU)."""
import torch
import torch.nn as nn


def _unit(mixed=True):
    from megalodon_b200.parallel.fsdp import FullyShardedDataParallel
    torch.manual_seed(0)
    lin = nn.Linear(48, 24)
    ref = nn.Linear(48, 24)
    ref.load_state_dict(lin.state_dict())
    unit = FullyShardedDataParallel(lin, mixed_precision=mixed, compute_dtype=torch.bfloat16,
                                    materialize_fp32_grads=False)
    return unit, ref


def test_micro_batches_accumulate_in_fp32():
    """Gradients of several backward passes before one optimiser step are summed in fp32 (each pass's
    own gradient is bf16, as in the reference's mixed-precision FSDP); a bf16 running sum would lose
    the low bits of every addend."""
    unit, ref = _unit()
    g = torch.Generator().manual_seed(1)
    parts = []
    for i in range(4):
        x = torch.randn(16, 48, generator=g) * (10.0 if i == 0 else 0.01)      # one large, three small
        unit(x.bfloat16()).float().pow(2).sum().backward()
        unit.finish_backward()
        ref.zero_grad()
        ref.to(torch.bfloat16)(x.bfloat16()).float().pow(2).sum().backward()
        parts.append(torch.cat([ref.weight.grad.flatten(), ref.bias.grad.flatten()]).float())
        ref.float()
    shard = unit.flat_param._grad_shard
    assert shard.dtype == torch.float32
    infos = {i.name: i for i in unit._infos}
    got = torch.cat([shard[infos[n].offset:infos[n].offset + infos[n].numel] for n in ("weight", "bias")])
    want = torch.stack(parts).sum(0)
    bf16_running = parts[0].bfloat16()
    for p in parts[1:]:
        bf16_running = (bf16_running + p.bfloat16())
    err_fp32 = (got - want).abs().max().item()
    err_bf16 = (bf16_running.float() - want).abs().max().item()
    assert err_fp32 <= 1e-3 * want.abs().max().item()
    assert err_fp32 < 0.1 * err_bf16, (err_fp32, err_bf16)


def test_chunk_group_sum_invalidates_the_norm_of_the_reduce_scatter():
    """A squared norm accumulated by a fused reduce-scatter describes the gradients before
    `grad_all_reduce()` changed them; clipping must not use it afterwards."""
    import torch.distributed as dist
    from unittest import mock
    unit, _ = _unit(mixed=False)
    unit(torch.randn(4, 48)).sum().backward()
    unit.finish_backward()
    unit._fused_sumsq = torch.tensor(123.0, dtype=torch.float64)
    unit._fused_sumsq_kind = "reduce_scatter"
    unit.chunk_parallel_world_size = 2            # pretend the chunk group holds replicas
    with mock.patch.object(dist, "all_reduce", lambda t, group=None, op=None: t.mul_(2.0)):
        unit.grad_all_reduce()
    assert unit._fused_sumsq is None


def test_flat_gradient_is_not_zero_filled_but_unused_parameters_and_gaps_end_up_zero():
    """The flat gradient buffer starts as uninitialised memory: the first contribution to a parameter is
    written, later ones are added, a parameter that received nothing and the gaps / padding between
    parameters are cleared before the gradients leave the unit."""
    from megalodon_b200.parallel.fsdp import FullyShardedDataParallel

    class Two(nn.Module):
        def __init__(self):
            super().__init__()
            self.used = nn.Linear(40, 24)
            self.unused = nn.Linear(24, 7)          # 7 * 24 + 7 elements: leaves an odd-sized tail

        def forward(self, x):
            return self.used(x) + self.used(x * 0.5)        # the weight is used twice: write, then add

    torch.manual_seed(0)
    mod = Two()
    ref = Two()
    ref.load_state_dict(mod.state_dict())
    unit = FullyShardedDataParallel(mod, mixed_precision=False, materialize_fp32_grads=False)
    x = torch.randn(8, 40)
    for _ in range(2):                                       # two iterations: the bookkeeping resets
        unit.zero_grad()
        unit(x).pow(2).sum().backward()
        unit.finish_backward()
        ref.zero_grad()
        ref(x).pow(2).sum().backward()
        shard = unit.flat_param._grad_shard
        assert torch.isfinite(shard).all()
        covered = torch.zeros(shard.numel(), dtype=torch.bool)
        for info in unit._infos:
            got = shard[info.offset:info.offset + info.numel].view(info.shape)
            covered[info.offset:info.offset + info.numel] = True
            want = dict(ref.named_parameters())[info.name].grad
            if want is None:
                assert bool((got == 0).all()), info.name
            else:
                assert torch.allclose(got, want, atol=1e-5, rtol=1e-5), info.name
        assert bool((shard[~covered] == 0).all())
