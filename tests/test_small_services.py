"""Small services without a test of their own: sharded grad scaler, fast_init, named scratch buffers, timers,
TP input broadcast, padded data gather over DP, pickled-object collectives (CPU / gloo)."""
import time

import torch

from dist_utils import run_ranks


def test_sharded_grad_scaler_skips_and_backs_off():
    from easyllm_b200.optim.grad_scaler import ShardedGradScaler
    p = torch.nn.Parameter(torch.tensor([1.0, 2.0]))
    opt = torch.optim.SGD([p], lr=0.5)
    sc = ShardedGradScaler(init_scale=8.0, growth_interval=2)
    sc.scale((p * torch.tensor([1.0, 3.0])).sum()).backward()
    assert p.grad.tolist() == [8.0, 24.0]
    sc.unscale_(opt)
    sc.unscale_(opt)                                   # second call in the same step is a no-op
    assert p.grad.tolist() == [1.0, 3.0]
    sc.step(opt); sc.update()
    assert p.detach().tolist() == [0.5, 0.5] and sc.get_scale() == 8.0
    opt.zero_grad()
    p.grad = torch.tensor([float("inf"), 1.0])
    before = p.detach().clone()
    assert sc.step(opt) is None                        # step skipped on overflow
    sc.update()
    assert torch.equal(p.detach(), before) and sc.get_scale() == 4.0
    for _ in range(2):                                 # two clean steps grow the scale again
        p.grad = torch.tensor([4.0, 4.0])
        sc.step(opt); sc.update()
    assert sc.get_scale() == 8.0
    other = ShardedGradScaler()
    other.load_state_dict(sc.state_dict())
    assert other.get_scale() == 8.0
    off = ShardedGradScaler(enabled=False)
    assert off.get_scale() == 1.0 and off.scale(torch.tensor(3.0)).item() == 3.0 and off.state_dict() == {}


def _scaler_rank(rank, world):
    from easyllm_b200.optim.grad_scaler import ShardedGradScaler
    p = torch.nn.Parameter(torch.ones(2))
    opt = torch.optim.SGD([p], lr=1.0)
    sc = ShardedGradScaler(init_scale=2.0)
    p.grad = torch.tensor([float("nan") if rank == 1 else 2.0, 2.0])
    out = sc.step(opt)
    sc.update()
    return out is None, p.detach().tolist(), sc.get_scale()


def test_sharded_grad_scaler_agrees_across_ranks():
    res = run_ranks(2, _scaler_rank)
    # only rank 1 overflowed, both ranks skip the step and halve the scale
    assert all(skipped and w == [1.0, 1.0] and s == 1.0 for skipped, w, s in res)


def test_fast_init_skips_allocation_and_random_init():
    from easyllm_b200.utils.fast_init import fast_init, materialize
    with fast_init():
        m = torch.nn.Sequential(torch.nn.Embedding(1000, 64), torch.nn.Linear(64, 64), torch.nn.LayerNorm(64))
    assert all(p.is_meta for p in m.parameters())
    m = materialize(m, "cpu")
    assert not any(p.is_meta for p in m.parameters()) and m[1].weight.shape == (64, 64)
    after = torch.nn.Linear(4, 4)                       # the patch is gone after the context
    assert not after.weight.is_meta and after.weight.abs().sum() > 0
    with fast_init(device="cpu"):
        t0 = time.time()
        big = torch.nn.Linear(2048, 2048)
        assert time.time() - t0 < 10.0 and not big.weight.is_meta


def test_global_memory_buffer_reuses_and_grows():
    from easyllm_b200.parallel.buffers import GlobalMemoryBuffer
    buf = GlobalMemoryBuffer()
    a = buf.get_tensor((4, 8), torch.float32, "ag", device="cpu")
    b = buf.get_tensor((2, 8), torch.float32, "ag", device="cpu")
    assert a.data_ptr() == b.data_ptr() and b.shape == (2, 8)
    c = buf.get_tensor((8, 8), torch.float32, "ag", device="cpu")
    assert c.numel() == 64
    d = buf.get_tensor((4, 8), torch.bfloat16, "ag", device="cpu")
    assert d.dtype == torch.bfloat16 and d.data_ptr() != c.data_ptr()
    buf.clear()
    assert buf._bufs == {}


def test_timers_and_memory_report():
    from easyllm_b200.utils.timers import Timers, report_memory
    t = Timers()
    t("step").start(); time.sleep(0.02); t("step").stop()
    t("step").start(); time.sleep(0.02); t("step").stop()
    e = t("step").elapsed(reset=False)
    assert 0.03 < e < 5.0
    assert t("step").elapsed() == e and t("step").elapsed() == 0.0       # reset by the second read
    lines = []
    report_memory("after step", printer=lines.append)
    assert len(lines) <= 1                              # one line on a GPU, nothing on a CPU-only host


def _tp_broadcast(rank, world):
    from easyllm_b200.parallel.data import broadcast_data
    from easyllm_b200.parallel.grid import get_grid, initialize_model_parallel
    from easyllm_b200.parallel.mappings import data_gather
    initialize_model_parallel(2, 1)                    # tp 2, dp 2
    g = get_grid()
    data = None
    if g.tp_rank == 0:
        data = {"input_ids": torch.arange(12).view(2, 6) + 100 * g.dp_rank, "labels": torch.arange(6).view(1, 6)}
    out = broadcast_data(["input_ids", "labels"], data, torch.int64)
    x = torch.full((g.dp_rank + 1, 3), float(g.dp_rank))
    parts = data_gather(x, dst=0)
    return (g.tp_rank, g.dp_rank, out["input_ids"].tolist(), out["labels"].tolist(),
            None if parts is None else [p.tolist() for p in parts])


def test_tp_input_broadcast_and_dp_padded_gather():
    res = run_ranks(4, _tp_broadcast)
    for tp_rank, dp_rank, ids, labels, parts in res:
        assert ids == (torch.arange(12).view(2, 6) + 100 * dp_rank).tolist() and labels == [list(range(6))]
        if dp_rank == 0:
            assert parts == [[[0.0] * 3], [[1.0] * 3, [1.0] * 3]]      # unpadded per-rank tensors on the destination
        else:
            assert parts is None


def _objects(rank, world):
    from easyllm_b200.parallel import hf_dist
    everyone = hf_dist.all_gather_object({"rank": rank, "payload": list(range(rank))})
    only0 = hf_dist.gather_pk(("r", rank))
    b = hf_dist.broadcast_object({"cfg": rank} if rank == 0 else None)
    return everyone, only0, b, hf_dist.get_rank(), hf_dist.get_world_size()


def test_pickled_object_collectives():
    res = run_ranks(3, _objects)
    for rank, (everyone, only0, b, r, w) in enumerate(res):
        assert [e["rank"] for e in everyone] == [0, 1, 2] and everyone[2]["payload"] == [0, 1]
        assert (only0 == [("r", 0), ("r", 1), ("r", 2)]) if rank == 0 else only0 is None
        assert b == {"cfg": 0} and r == rank and w == 3


def test_storage_helper_local_paths_pointer_files_and_fake_remote(tmp_path, monkeypatch):
    import json
    import pytest
    from easyllm_b200.utils.petrel_helper import PetrelHelper, get_ceph_path
    # local paths: save creates folders, load / exists / listdir / open / load_json work on files
    target = tmp_path / "a" / "b" / "w.pt"
    PetrelHelper.save({"w": torch.arange(3)}, str(target))
    assert PetrelHelper.exists(str(target)) and PetrelHelper.listdir(str(tmp_path / "a" / "b")) == ["w.pt"]
    assert PetrelHelper.load(str(target))["w"].tolist() == [0, 1, 2]
    (tmp_path / "c.json").write_text(json.dumps({"k": 1}))
    assert PetrelHelper.load_json(str(tmp_path / "c.json")) == {"k": 1}
    # pointer files: `<path>.ceph` / `<path>.ini` name the real location on their first line
    (tmp_path / "ckpt.ceph").write_text(str(target) + "\nsecond line ignored\n")
    assert PetrelHelper.resolve(str(tmp_path / "ckpt")) == str(target)
    assert PetrelHelper.load(str(tmp_path / "ckpt"))["w"].tolist() == [0, 1, 2]
    (tmp_path / "link.ini").write_text(str(tmp_path / "c.json"))
    assert PetrelHelper.load_json(str(tmp_path / "link.ini")) == {"k": 1}
    assert PetrelHelper.resolve(str(tmp_path / "plain")) == str(tmp_path / "plain")
    # bucket prefixing
    assert get_ceph_path("./ckpt/step1", "s3://bucket/run/") == "s3://bucket/run/ckpt/step1"
    assert get_ceph_path("ckpt/step1", "") == "ckpt/step1"
    monkeypatch.setenv("CEPHBUCKET", "s3://b")
    assert get_ceph_path("/x/y") == "s3://b/x/y"
    # s3:// without the SDK is a clear error; with a client (a fake here) every call goes through it
    assert PetrelHelper.is_remote("s3://bucket/x") and not PetrelHelper.is_remote(str(target))
    monkeypatch.setattr(PetrelHelper, "_client", None)
    with pytest.raises(RuntimeError, match="petrel_client"):
        PetrelHelper.load("s3://bucket/x.pt")

    class FakeClient:
        def __init__(self):
            self.store = {}

        def put(self, k, v):
            self.store[k] = v

        def get(self, k):
            return self.store[k]

        def contains(self, k):
            return k in self.store

        def list(self, prefix):
            return [k[len(prefix):] for k in self.store if k.startswith(prefix)]
    fake = FakeClient()
    monkeypatch.setattr(PetrelHelper, "_client", fake)
    PetrelHelper.save({"w": torch.ones(2)}, "s3://bucket/run/w.pt")
    assert PetrelHelper.exists("s3://bucket/run/w.pt") and PetrelHelper.listdir("s3://bucket/run/") == ["w.pt"]
    assert PetrelHelper.load("s3://bucket/run/w.pt")["w"].tolist() == [1.0, 1.0]
    fake.put("s3://bucket/c.json", b'{"r": 2}')
    assert PetrelHelper.load_json("s3://bucket/c.json") == {"r": 2}
    (tmp_path / "remote.ceph").write_text("s3://bucket/run/w.pt")
    assert PetrelHelper.load(str(tmp_path / "remote"))["w"].tolist() == [1.0, 1.0]


def test_download_tool_follows_pointer_files(tmp_path, monkeypatch):
    """``tools/download_fromceph.py`` on a folder of ``.ceph`` pointer files and plain files, with a fake remote."""
    import importlib.util
    import os
    from easyllm_b200.utils.petrel_helper import PetrelHelper

    class Fake:
        store = {"s3://b/run/layer_01.pt": b"REMOTE-BYTES"}

        def get(self, k):
            return self.store[k]

        def list(self, prefix):
            return [k[len(prefix):] for k in self.store if k.startswith(prefix)]
    monkeypatch.setattr(PetrelHelper, "_client", Fake())
    src = tmp_path / "ck"
    src.mkdir()
    (src / "layer_01.pt.ceph").write_text("s3://b/run/layer_01.pt\n")
    (src / "latest").write_text("global_step1")
    spec = importlib.util.spec_from_file_location("dl", os.path.join(os.path.dirname(__file__), "..", "tools",
                                                                     "download_fromceph.py"))
    tool = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(tool)
    tool.main(["--src", str(src), "--dst", str(tmp_path / "out")])
    assert (tmp_path / "out" / "layer_01.pt").read_bytes() == b"REMOTE-BYTES"
    assert (tmp_path / "out" / "latest").read_text() == "global_step1"
    tool.main(["--src", "s3://b/run/", "--dst", str(tmp_path / "out2")])
    assert (tmp_path / "out2" / "layer_01.pt").read_bytes() == b"REMOTE-BYTES"
