"""Host-buffer entry point: the same step with inputs and output in host memory, synchronous and pipelined
(sync=0, two staging slots in the library, results collected with host_sync)."""
import pytest
import torch

import workloads

pytestmark = pytest.mark.gpu


def _workloads(pkg, n):
    wl = workloads
    cfg = wl.DecodeConfig("host", 6, 16, 2, 128, torch.bfloat16, "fp8", 64, 200, 1500, True, 77)
    return cfg, [wl.build_workload(cfg, "cpu", seed_offset=i) for i in range(n)]


def _device_result(pkg, cfg, w_cpu):
    wl = workloads
    w = wl.to_device(w_cpu, "cuda:0")
    plugin = wl.make_plugin(cfg, 0)
    out = wl.run_step(plugin, w)
    torch.cuda.synchronize()
    plugin.close()
    return out.cpu(), w.pool.cpu()


@pytest.mark.parametrize("pipelined", [False, True])
def test_host_path_matches_the_device_path(pkg, pipelined):
    wl = workloads
    cfg, cpu = _workloads(pkg, 5)
    want = [_device_result(pkg, cfg, w) for w in cpu]
    dev = [wl.to_device(w, "cuda:0") for w in cpu]   # pools and scales live on the device
    plugin = wl.make_plugin(cfg, 0)
    pin = lambda t: t.cpu().pin_memory()
    outs = [torch.zeros(cfg.batch, cfg.num_heads * cfg.head_size, dtype=cfg.dtype).pin_memory() for _ in dev]
    keep = []
    try:
        for w, o in zip(dev, outs):
            args = (pin(w.qkv), pin(w.sequence_length), w.host_past_key_value_lengths, pin(w.kv_cache_block_pointers))
            keep.append(args)
            plugin.enqueue_generation_host(*args, w.kv_orig_quant_scale, w.kv_quant_orig_scale, o,
                                           max_attention_window=w.max_blocks_per_seq * cfg.tokens_per_block,
                                           sync=not pipelined)
            if not pipelined:
                assert torch.equal(o, want[len(keep) - 1][0])  # in host memory when the call returns
        plugin.host_sync()
        assert plugin.device_status() == 0
        for (o_want, pool_want), o, w in zip(want, outs, dev):
            assert torch.equal(o, o_want)
            assert torch.equal(w.pool.cpu(), pool_want)
    finally:
        plugin.close()
