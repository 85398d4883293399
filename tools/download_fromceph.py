"""Copy a checkpoint directory from remote (s3://, via ``.ceph`` pointer files) to local disk
(tools/download_fromceph.py of the reference; pointer-file convention of llm/utils/tools/petrel_helper.py:127-135)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main(argv=None):
    from easyllm_b200.utils.petrel_helper import PetrelHelper
    p = argparse.ArgumentParser()
    p.add_argument("--src", required=True, help="directory of .ceph pointer files, or an s3:// prefix")
    p.add_argument("--dst", required=True)
    a = p.parse_args(argv)
    os.makedirs(a.dst, exist_ok=True)
    for name in PetrelHelper.listdir(a.src):
        src = os.path.join(a.src, name) if not PetrelHelper.is_remote(a.src) else a.src.rstrip("/") + "/" + name
        target = os.path.join(a.dst, name[:-5] if name.endswith(".ceph") else name)
        with PetrelHelper.open(src, "rb") as f, open(target, "wb") as out:
            out.write(f.read())
        print("fetched", target)


if __name__ == "__main__":
    main()
