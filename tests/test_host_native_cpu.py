"""Host-only native classes (no GPU needed): Config, size hints, the low-latency layout and the arena allocator."""
import random

import pytest

from deepep_efa_b200 import _ext, Config, Buffer

C = _ext.load()


def test_config_signature_and_validation():
    c = Config(20, 6, 256, 6, 128)
    assert (c.num_sms, c.num_max_nvl_chunked_send_tokens, c.num_max_nvl_chunked_recv_tokens) == (20, 6, 256)
    assert c.num_max_rdma_chunked_recv_tokens % c.num_max_rdma_chunked_send_tokens == 0
    with pytest.raises(ValueError):
        Config(20, 256, 6, 6, 128)
    assert c.get_rdma_buffer_size_hint(7168 * 2, 8) == 0
    h8 = c.get_nvl_buffer_size_hint(7168 * 2, 8)
    h2 = c.get_nvl_buffer_size_hint(7168 * 2, 2)
    assert h8 > h2 > C.CONTROL_BYTES and h8 % 128 == 0
    for r in (1, 2, 4, 8):
        assert Buffer.get_dispatch_config(r).num_sms > 0 and Buffer.get_combine_config(r).num_sms > 0


def test_low_latency_size_hint_monotone():
    a = Buffer.get_low_latency_rdma_size_hint(128, 7168, 8, 256)
    b = Buffer.get_low_latency_rdma_size_hint(256, 7168, 8, 256)
    assert b > a > 0 and a % 128 == 0
    with pytest.raises(ValueError):
        Buffer.get_low_latency_rdma_size_hint(128, 7168, 8, 250)


def test_arena_alloc_free_coalesce():
    a = C.Arena(4096, 1 << 20, 1024)
    assert a.capacity == 1 << 20
    blocks = [a.alloc(1000) for _ in range(8)]
    assert len(set(blocks)) == 8 and all(b % 1024 == 0 and b >= 4096 for b in blocks)
    assert a.in_use == 8 * 1024
    for b in blocks[::2]:
        a.free(b)
    assert a.num_free_blocks >= 4
    for b in blocks[1::2]:
        a.free(b)
    assert a.in_use == 0 and a.num_free_blocks == 1 and a.largest_free == 1 << 20
    with pytest.raises(RuntimeError):
        a.free(blocks[0])
    assert a.alloc(2 << 20) == -1


def test_arena_random_stress():
    rng = random.Random(0)
    a = C.Arena(0, 1 << 22, 256)
    live = {}
    for _ in range(2000):
        if live and rng.random() < 0.5:
            off = rng.choice(list(live))
            a.free(off)
            del live[off]
        else:
            n = rng.randint(1, 40000)
            off = a.alloc(n)
            if off >= 0:
                for o, s in live.items():
                    assert off + n <= o or o + s <= off, "overlap"
                live[off] = n
    for off in list(live):
        a.free(off)
    assert a.in_use == 0 and a.num_free_blocks == 1


def test_low_latency_layout_class():
    import deepep_efa_b200 as ep
    lay = ep.LowLatencyLayout(C.CONTROL_BYTES, 128, 7168, 8, 256)
    offs = [lay.counts_off, lay.recv_x_off, lay.recv_scales_off, lay.recv_src_info_off, lay.combine_stage_off, lay.combine_src_off]
    flat = sorted(o for pair in offs for o in pair)
    assert flat[0] == C.CONTROL_BYTES and all(b > a for a, b in zip(flat, flat[1:])) and all(o % 1024 == 0 for o in flat)
    assert lay.total_bytes + C.CONTROL_BYTES <= ep.Buffer.get_low_latency_rdma_size_hint(128, 7168, 8, 256) + 128
    # recv_x is sized for BF16 dispatch: L * N * hidden * 2 bytes per parity
    assert lay.recv_scales_off[0] - lay.recv_x_off[0] >= 32 * 1024 * 7168 * 2
