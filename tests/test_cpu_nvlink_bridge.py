"""``NVLinkBroadcastBridge`` without a GPU: a stand-in for the symmetric memory (one byte window per rank, addresses that
encode the rank) and for the ``cast_broadcast`` kernel, so that the publish / join / import / acknowledge protocol, the
dtype cast, the packed layout, the capacity check and tamper detection run as plain host code on several "ranks"."""

import types

import pytest
import torch

from rl_engine.executors.bridge import (
    NVLinkBroadcastBridge, WeightBridgeUnavailableError, WeightManifestValidationError, WeightUpdateRejectedError,
)

SHIFT = 44
DTYPE_OF_CODE = {0: torch.float32, 1: torch.bfloat16, 2: torch.float16}


class FakeWorld:
    """``world`` byte windows and the barrier bookkeeping shared by the fake memories of all ranks."""

    def __init__(self, world: int, nbytes: int) -> None:
        self.windows = [torch.zeros(nbytes, dtype=torch.uint8) for _ in range(world)]
        self.barriers = [0] * world
        self.launches = 0

    def memory(self, rank: int):
        outer = self

        class Window:
            def __init__(self, offset, n):
                self.local = outer.windows[rank][offset : offset + n]
                self.ptrs = [((r + 1) << SHIFT) + offset for r in range(len(outer.windows))]

        class Memory:
            world = len(outer.windows)

            def __init__(self):
                self.rank = rank
                self._cursor = 0

            def alloc(self, shape, dtype):
                nbytes = int(shape[0]) * torch.empty((), dtype=dtype).element_size()
                start = (self._cursor + 255) // 256 * 256
                w = Window(start, nbytes)
                w.local = w.local.view(dtype)
                self._cursor = start + nbytes
                return w

            def barrier(self, channel: int = 0):
                outer.barriers[rank] += 1

        return Memory()

    def cast_broadcast(self, src, addrs, code):
        """What the kernel does: read ``src`` once, cast, store into every rank's window at the given address."""
        self.launches += 1
        data = src.reshape(-1).to(DTYPE_OF_CODE[code]).contiguous().view(torch.uint8)
        for addr in addrs:
            rank, offset = (addr >> SHIFT) - 1, addr & ((1 << SHIFT) - 1)
            self.windows[rank][offset : offset + data.numel()] = data


@pytest.fixture
def fake_world(monkeypatch):
    world = FakeWorld(3, 1 << 16)
    import rl_engine.kernels.ops.base as base

    monkeypatch.setattr(base, "require_ext", lambda: types.SimpleNamespace(cast_broadcast=world.cast_broadcast))
    return world


def _model():
    torch.manual_seed(0)
    m = torch.nn.Sequential(torch.nn.Linear(6, 4), torch.nn.Linear(4, 3, bias=False))
    m.register_buffer("steps", torch.tensor([7, 9], dtype=torch.int64))
    m.register_buffer("flag", torch.tensor([True, False, True]))
    return m


def test_publish_join_import_acknowledge_on_three_ranks(fake_world):
    bridges = [NVLinkBroadcastBridge(fake_world.memory(r), 1 << 15, target_dtype=torch.bfloat16, relay=False)
               for r in range(3)]
    model = _model()
    manifest = bridges[0].publish(model, weight_version=1)
    for b in bridges[1:]:
        b.join_publish()
    assert fake_world.barriers == [2, 2, 2]                      # window free / window complete, on every rank
    # one cast per tensor into the publisher's own window, then the whole window to the two peers in one transfer
    assert manifest.transport == "nvlink-broadcast" and fake_world.launches == len(manifest.tensors) + 1 == 6
    block = manifest.metadata["weight_bridge"]
    assert block["world_size"] == 3 and all(e["offset"] % 256 == 0 for e in block["tensors"].values())
    for rank, bridge in enumerate(bridges):
        got = bridge.import_update(manifest)
        assert got["0.weight"].dtype == torch.bfloat16            # floating tensors were cast on the way
        assert torch.equal(got["0.weight"], model[0].weight.detach().to(torch.bfloat16))
        assert torch.equal(got["steps"], model.steps) and torch.equal(got["flag"].bool(), model.flag)
        # zero copy: the tensors are views of this rank's window
        assert got["1.weight"].untyped_storage().data_ptr() == fake_world.windows[rank].untyped_storage().data_ptr()
        bridge.acknowledge(manifest.update_id)
        assert bridge.active_weight_version == 1 and bridge.update_status(manifest.update_id) == "acknowledged"
    # the next version overwrites the windows in place; versions must increase
    with torch.no_grad():
        model[0].weight.mul_(2.0)
    with pytest.raises(WeightManifestValidationError):
        bridges[0].publish(model, weight_version=1)
    second = bridges[0].publish(model, weight_version=2)
    bridges[1].join_publish()
    bridges[2].join_publish()
    assert torch.equal(bridges[2].import_update(second)["0.weight"], model[0].weight.detach().to(torch.bfloat16))


def test_relay_mode_fills_every_window_with_less_traffic_from_the_source(fake_world):
    """Relay: the source stores into its own window, sends slice j to rank j, every rank forwards its slice.  The fake
    kernel cannot run concurrently, so the ranks' steps are interleaved by hand in barrier order."""
    direct_world = FakeWorld(3, 1 << 16)
    model = _model()
    bridges = [NVLinkBroadcastBridge(fake_world.memory(r), 1 << 15, target_dtype=torch.bfloat16) for r in range(3)]
    assert all(b.relay for b in bridges)
    sent = []
    real = fake_world.cast_broadcast

    def counting(src, addrs, code):
        sent.append((src.numel() * DTYPE_OF_CODE[code].itemsize, [(a >> SHIFT) - 1 for a in addrs]))
        real(src, addrs, code)

    import rl_engine.kernels.ops.base as base

    base.require_ext = lambda: types.SimpleNamespace(cast_broadcast=counting)
    manifest = bridges[0].publish(model, weight_version=1)        # hop 1 + the source's part of hop 2
    for b in bridges[1:]:
        b.join_publish()                                          # hop 2 of the consumers
    assert fake_world.barriers == [3, 3, 3] and manifest.metadata["weight_bridge"]["relay"] is True
    total = manifest.metadata["weight_bridge"]["requested_nbytes"]
    windows = [w[: total].clone() for w in fake_world.windows]
    assert torch.equal(windows[0], windows[1]) and torch.equal(windows[0], windows[2])
    for bridge in bridges:
        got = bridge.import_update(manifest)
        assert torch.equal(got["1.weight"], model[1].weight.detach().to(torch.bfloat16))
        bridge.acknowledge(manifest.update_id)
    # bytes that left the source for OTHER ranks: about one copy of the update (plus the 64-byte header per peer),
    # where direct mode sends one copy per peer
    from_source = sum(nbytes * len([r for r in ranks if r != 0]) for nbytes, ranks in sent[: sent.index(sent[-2])])
    assert from_source <= total + 2 * 64 + 3 * 256
    # same bytes as direct mode
    base.require_ext = lambda: types.SimpleNamespace(cast_broadcast=direct_world.cast_broadcast)
    direct = [NVLinkBroadcastBridge(direct_world.memory(r), 1 << 15, target_dtype=torch.bfloat16, relay=False)
              for r in range(3)]
    direct[0].publish(model, weight_version=1)
    assert torch.equal(direct_world.windows[2][: total], windows[2])


def test_kernel_store_mode_casts_straight_into_every_window(fake_world):
    """``stores="kernel"``: one fused cast + peer-store launch per tensor writes all windows (direct mode), nothing is
    staged; the resulting windows and manifests equal those of the copy-engine mode."""
    model = _model()
    fused = [NVLinkBroadcastBridge(fake_world.memory(r), 1 << 15, target_dtype=torch.bfloat16, relay=False, stores="kernel")
             for r in range(3)]
    manifest = fused[0].publish(model, weight_version=1)
    for b in fused[1:]:
        b.join_publish()
    assert fake_world.launches == len(manifest.tensors) == 5
    other = FakeWorld(3, 1 << 16)
    import rl_engine.kernels.ops.base as base

    base.require_ext = lambda: types.SimpleNamespace(cast_broadcast=other.cast_broadcast)
    staged = [NVLinkBroadcastBridge(other.memory(r), 1 << 15, target_dtype=torch.bfloat16, relay=False) for r in range(3)]
    staged[0].publish(model, weight_version=1)
    total = manifest.metadata["weight_bridge"]["requested_nbytes"]
    for r in range(3):
        assert torch.equal(fake_world.windows[r][:total], other.windows[r][:total])
    # relay mode on the same engine: own window first, then slices and forwards by the same kernel
    relay_world = FakeWorld(3, 1 << 16)
    base.require_ext = lambda: types.SimpleNamespace(cast_broadcast=relay_world.cast_broadcast)
    relayed = [NVLinkBroadcastBridge(relay_world.memory(r), 1 << 15, target_dtype=torch.bfloat16, relay=True, stores="kernel")
               for r in range(3)]
    relayed[0].publish(model, weight_version=1)
    for b in relayed[1:]:
        b.join_publish()
    for r in range(3):
        assert torch.equal(relay_world.windows[r][:total], other.windows[r][:total])
    with pytest.raises(ValueError):
        NVLinkBroadcastBridge(fake_world.memory(0), 1 << 10, stores="nccl")


def test_hop_two_destinations_are_rotated_and_skip_the_source(fake_world):
    """Every rank forwards its slice to all ranks that still miss it, starting with its right-hand neighbour, so that
    the k-th transfers of the ranks do not all land on one GPU."""
    world = 3
    bridges = [NVLinkBroadcastBridge(fake_world.memory(r), 1 << 15) for r in range(world)]
    source = 0
    orders = [b._forward_order(source) for b in bridges]
    assert orders[0] == [1, 2]                      # the source forwards its own slice to everybody else
    assert orders[1] == [2] and orders[2] == [1]    # consumers skip themselves and the source
    big = FakeWorld(8, 1 << 12)
    eight = [NVLinkBroadcastBridge(big.memory(r), 1 << 10) for r in range(8)]
    firsts = [b._forward_order(0)[0] for b in eight]
    assert len(set(firsts)) >= 7                    # first transfers go to (almost) all different ranks
    for r, b in enumerate(eight):
        order = b._forward_order(0)
        assert r not in order and len(order) == len(set(order)) == (7 if r == 0 else 6)


def test_sync_is_one_collective_call(fake_world):
    bridges = [NVLinkBroadcastBridge(fake_world.memory(r), 1 << 15, relay=False) for r in range(3)]
    model = _model()
    shipped = {}

    def fake_dist(rank):
        def broadcast_object_list(box, src=0, group=None):
            if rank == src:
                shipped["manifest"] = box[0]
            else:
                box[0] = shipped["manifest"]

        return types.SimpleNamespace(broadcast_object_list=broadcast_object_list)

    results = [bridges[r].sync(model if r == 0 else None, weight_version=4, dist=fake_dist(r)) for r in range(3)]
    for rank, (manifest, tensors) in enumerate(results):
        assert manifest.weight_version == 4 and torch.equal(tensors["0.bias"], model[0].bias.detach())
        assert bridges[rank].active_weight_version == 4
    assert fake_world.barriers == [2, 2, 2]


def test_capacity_tampering_and_unknown_manifests(fake_world):
    small = NVLinkBroadcastBridge(fake_world.memory(0), 64)
    with pytest.raises(WeightBridgeUnavailableError, match="window holds 256"):
        small.publish(_model(), weight_version=1)
    bridge = NVLinkBroadcastBridge(fake_world.memory(0), 1 << 14)
    model = _model()
    manifest = bridge.publish(model, weight_version=1)
    tensors = bridge.import_update(manifest)
    tensors["0.weight"].view(-1)[0] += 1.0                        # someone scribbles into the window
    with pytest.raises(WeightManifestValidationError, match="checksum"):
        bridge.acknowledge(manifest.update_id)
    other = NVLinkBroadcastBridge(fake_world.memory(1), 1 << 14)
    local = types.SimpleNamespace(**{**manifest.__dict__, "metadata": {"weight_bridge": {"format": "something-else"}}})
    with pytest.raises(WeightUpdateRejectedError):
        other.import_update(local)
