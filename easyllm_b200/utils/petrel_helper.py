"""Remote-storage helper with a local-filesystem fallback.

Parity: llm/utils/tools/petrel_helper.py:9-184 — ``s3://`` paths go through the Petrel (Ceph) SDK
when it is importable and ``PETRELPATH`` names its config; ``.ceph`` / ``.ini`` pointer files
hold the remote location of a checkpoint.  Without the SDK every call works on local paths and
``s3://`` raises a clear error.  ``CheckpointManager`` (async_helper.py:29-93) snapshots tensors
to host memory and writes them from a background thread so training does not wait on storage.
"""
from __future__ import annotations

import io
import json
import os
import threading

import torch


class PetrelHelper:
    _client = None

    @classmethod
    def client(cls):
        if cls._client is None:
            try:
                from petrel_client.client import Client
            except ImportError as e:
                raise RuntimeError("s3:// paths need the petrel_client SDK (not installed); use a local path") from e
            cls._client = Client(os.environ.get("PETRELPATH", "~/petreloss.conf"))
        return cls._client

    @staticmethod
    def is_remote(path):
        return isinstance(path, str) and path.startswith("s3://")

    @staticmethod
    def resolve(path):
        """Follow ``.ceph`` / ``.ini`` pointer files to the location they name."""
        for ext in (".ceph", ".ini"):
            p = path if path.endswith(ext) else path + ext
            if os.path.exists(p):
                with open(p) as f:
                    return f.readline().strip()
        return path

    @classmethod
    def open(cls, path, mode="r"):
        path = cls.resolve(path)
        if cls.is_remote(path):
            data = cls.client().get(path)
            return io.StringIO(data.decode()) if "b" not in mode else io.BytesIO(data)
        return open(path, mode)

    @classmethod
    def load_json(cls, path):
        with cls.open(path) as f:
            return json.load(f)

    @classmethod
    def load(cls, path, **kw):
        path = cls.resolve(path)
        if cls.is_remote(path):
            return torch.load(io.BytesIO(cls.client().get(path)), **kw)
        return torch.load(path, **kw)

    @classmethod
    def save(cls, obj, path):
        if cls.is_remote(path):
            buf = io.BytesIO()
            torch.save(obj, buf)
            cls.client().put(path, buf.getvalue())
        else:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
            torch.save(obj, path)

    @classmethod
    def listdir(cls, path):
        if cls.is_remote(path):
            return list(cls.client().list(path))
        return os.listdir(path)

    @classmethod
    def exists(cls, path):
        if cls.is_remote(path):
            return cls.client().contains(path)
        return os.path.exists(path)


def get_ceph_path(path, bucket=None):
    bucket = bucket if bucket is not None else os.environ.get("CEPHBUCKET", "")
    if not bucket:
        return path
    return bucket.rstrip("/") + "/" + path.lstrip("./").lstrip("/")


class CheckpointManager:
    """Asynchronous checkpoint writer: ``save(state_dict, path)`` copies tensors to host memory on
    the caller's stream and returns; a worker thread serialises them.  ``wait()`` joins."""

    def __init__(self, max_pending=1):
        self._threads = []
        self.max_pending = max_pending

    @staticmethod
    def _to_cpu(obj):
        if torch.is_tensor(obj):
            return obj.detach().to("cpu", non_blocking=False).clone()
        if isinstance(obj, dict):
            return {k: CheckpointManager._to_cpu(v) for k, v in obj.items()}
        if isinstance(obj, (list, tuple)):
            return type(obj)(CheckpointManager._to_cpu(v) for v in obj)
        return obj

    def save(self, state, path):
        self._threads = [t for t in self._threads if t.is_alive()]
        while len(self._threads) >= self.max_pending:
            self._threads.pop(0).join()
        snap = self._to_cpu(state)

        def work():
            tmp = path + ".tmp"
            PetrelHelper.save(snap, tmp)
            if not PetrelHelper.is_remote(path):
                os.replace(tmp, path)
        t = threading.Thread(target=work, daemon=True)
        t.start()
        self._threads.append(t)

    def wait(self):
        for t in self._threads:
            t.join()
        self._threads = []
