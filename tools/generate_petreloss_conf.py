"""Write a ``petreloss.conf`` for the Petrel (Ceph) SDK from command-line credentials
(tools/generate_petreloss_conf.py of the reference)."""
import argparse
import os


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--access_key", required=True)
    p.add_argument("--secret_key", required=True)
    p.add_argument("--host_base", required=True)
    p.add_argument("--cluster", default="default")
    p.add_argument("--out", default=os.path.expanduser("~/petreloss.conf"))
    a = p.parse_args(argv)
    with open(a.out, "w") as f:
        f.write("[DEFAULT]\ndefault_cluster = {c}\n\n[{c}]\naccess_key = {ak}\nsecret_key = {sk}\nhost_base = {hb}\n"
                .format(c=a.cluster, ak=a.access_key, sk=a.secret_key, hb=a.host_base))
    print("wrote", a.out)


if __name__ == "__main__":
    main()
