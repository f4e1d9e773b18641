"""The launchers' host-side choices (tile widths, split counts, bounds of the expert layout), which need no device."""
import itertools
import random

from turboquant_cpp_b200.kernels import attention as KA
from turboquant_cpp_b200.kernels import gemm_tc as KT
from turboquant_cpp_b200.kernels import moe as KM


def test_max_tiles_bounds_every_routing():
    """However n_pairs rows fall on the experts, the row tiles (each expert's rows cut into tiles of at most
    tile_rows, never across two experts) are at most max_tiles."""
    rng = random.Random(0)
    for _ in range(300):
        E, tile = rng.randint(1, 12), rng.choice([1, 2, 3, 16, 64])
        P = rng.randint(1, 200)
        counts = [0] * E
        for _ in range(P):
            counts[rng.randrange(E) if rng.random() < 0.7 else 0] += 1
        tiles = sum(-(-c // tile) for c in counts)
        assert tiles <= KM.max_tiles(P, E, tile)
    assert KM.max_tiles(5, 60, 16) == 5 and KM.max_tiles(8192, 60, 256) == 92


def test_token_tile_is_a_kernel_width_and_grows_with_the_rows():
    last = 0
    for rows in range(1, 5000, 7):
        bn = KT.token_tile_for(rows, 1)
        assert bn in KT.TOKEN_TILES and bn >= last
        last = bn
    assert KT.token_tile_for(32, 60) == 16            # a decode step: one or two rows per expert
    assert KT.token_tile_for(8192, 60) == 256         # a 2,048-token prompt, top-4 of 60: about 137 rows each
    assert KT.token_tile_for(10 ** 6, 1) == KT.TOKEN_TILES[-1]


def test_split_counts_fit_the_kernel_and_fill_a_wave():
    for tokens, heads in itertools.product([1, 2, 3, 8, 31, 64, 200, 1000, 5000], [1, 2, 4, 16, 28]):
        s = KA.splits_for(tokens, heads)
        assert 1 <= s <= 16
        rows = tokens * heads
        if rows * 2 <= KA.RESIDENT_CTAS:               # few rows: as many ranges as fit one wave, 16 at most
            assert s == min(16, KA.RESIDENT_CTAS // rows)
        if rows >= 4 * KA.RESIDENT_CTAS:
            assert s == 1
    assert KA.splits_for(8, 16) == 4 and KA.splits_for(64, 16) == 4 and KA.splits_for(1, 16) == 16


def test_small_router_limits():
    assert KM.router_small_usable(8, 4, 60, 2048) and KM.router_small_pays(8, 4, 60, 2048)
    assert KM.router_small_usable(64, 4, 60, 2048) and not KM.router_small_pays(64, 4, 60, 2048)   # 256 pairs: not worth it
    assert not KM.router_small_usable(200, 4, 60, 2048)            # more than 512 pairs
    assert not KM.router_small_usable(1, 1, 1024, 64)              # more experts than the scan has threads
    assert not KM.router_small_usable(1, 1, 8, 8192)               # the row and the logits do not fit shared memory
    assert KM.align_chunk(100) == 512 and KM.align_chunk(256 * 256 * 3) == 768


def test_attention_head_sizes():
    import pytest
    for hd in range(16, 257, 16):
        KA.check_head_dim(hd)
    for hd in (0, 8, 24, 100, 272):
        with pytest.raises(KA.KernelError):
            KA.check_head_dim(hd)
    assert KA.split_usable(16, 16, 128, 64) and KA.split_usable(28, 4, 128, 64)
    assert KA.split_usable(16, 1, 128, 64)             # 16 query heads per KV head: shared out over two CTAs
    assert not KA.split_usable(4, 4, 48, 64)           # head size 48: the exact kernel takes it
    assert KA.prefill_usable(__import__("torch").bfloat16, 128, 64) and not KA.prefill_usable(__import__("torch").float32, 128, 64)


def test_shares_of_the_shared_down_projection():
    """The sizes of the two real models: whole from the batch on where sharing it out was measured to cost, in shares
    below; prompts (wide token tiles) never."""
    from turboquant_cpp_b200.parts.moe_ffn import experts_touched, shared_down_shares
    a = dict(n_experts=60, top_k=4, intermediate=1408, shared_intermediate=5632, hidden=2048, sms=148)
    b = dict(n_experts=64, top_k=8, intermediate=2560, shared_intermediate=20480, hidden=3584, sms=148)
    shares = lambda m, T, first=False: shared_down_shares(T, token_tile=KT.token_tile_for(T, 1), router_first=first, **m)
    assert shares(a, 1) > 4 and shares(a, 2) > 4                    # the longer chain of the layer: over the whole GPU
    assert [shares(a, T) for T in (3, 4, 5)] == [2, 2, 2]
    assert [shares(a, T) for T in (6, 8, 12)] == [1, 1, 1]
    assert shares(a, 16, first=True) > 1                            # the router ran first: beside the routed experts, shared out
    assert shares(b, 1) > 8 and [shares(b, T) for T in (3, 4, 6)] == [4, 4, 4] and shares(b, 7) == 1
    assert shares(a, 2048) == 1 and shares(b, 300) == 1
    assert shared_down_shares(4, 8, 2, 64, 128, 64, 16, 148, False) == 1        # a tiny model: too short a K to share out
    assert abs(experts_touched(1, 60, 4) - 4) < 1e-9 and 25 < experts_touched(8, 60, 4) < 26
    assert experts_touched(10 ** 6, 60, 4) <= 60


def test_when_the_shared_expert_rides_in_the_routed_launches():
    from turboquant_cpp_b200.parts.moe_ffn import shared_rides_with_routed
    assert [shared_rides_with_routed(T, 5632, 148) for T in (768, 1024, 1536, 2048, 8192)] == [True, True, True, False, False]
    assert not shared_rides_with_routed(512, 20480, 148)            # the larger model's shared expert fills the GPU sooner
