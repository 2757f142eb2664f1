"""Generates tests/golden/<case>.npz by running the UNMODIFIED reference (oracle/_ref/libmyea_ref.so, built by
oracle/build_ref.sh from the reference checkout) on every case of tests/cases.py.  Run from the repository root:

    python tests/golden/make_golden.py [case ...]
    python tests/golden/make_golden.py --pre-training      (the autoencoder pre-training fixtures)

The fixtures hold the reference's derivatives, losses, updated parameters, first moments, running normalization
statistics, last-layer outputs, index map and sizes in float32 / float64 / int64; inputs are regenerated from seeds by
myea_b200/workloads.py and guarded by a checksum stored beside the results.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from oracle import ref  # noqa: E402


def input_checksum(wl, net):
    X, Y = wl.batch()
    p = wl.parameters(net)
    return np.array([float(np.abs(X).sum(dtype=np.float64)), float(np.abs(Y).sum(dtype=np.float64)), float(np.abs(p).sum(dtype=np.float64))])


PRE_TRAINING = {"autoencoder_pre_training": cases.capi.DROP_NONE, "autoencoder_pre_training_dropout": cases.capi.DROP_BERNOULLI_INVERTED}


def pre_training():
    """tests/golden/autoencoder_pre_training*.npz: the pre-training levels 1, 2 and the whole network, two steps each"""
    for name, drop in PRE_TRAINING.items():
        wl = cases.autoencoder_case(drop)
        net = ref.RefNet(wl.desc, wl.opt, threads=1)
        out = cases.run_pre_training(net, wl)
        net.close()
        arrays = {k: np.asarray(v, np.float64 if k.endswith("loss") else np.float32) for k, v in out.items()}
        path = os.path.join(ROOT, "tests", "golden", name + ".npz")
        np.savez_compressed(path, **arrays)
        print("%-32s %6.1f KiB" % (name, os.path.getsize(path) / 1024.0))


def main():
    if sys.argv[1:] == ["--pre-training"]:
        return pre_training()
    names = sys.argv[1:] or sorted(cases.CASES)
    for name in names:
        wl = cases.CASES[name]()
        net = ref.RefNet(wl.desc, wl.opt, threads=1)
        out = cases.run_steps(net, wl)
        out["input_checksum"] = input_checksum(wl, net)
        net.close()
        shake = out.pop("shake")
        for it, draws in enumerate(shake):          # the reference's own ShakeDrop draws, so that they can be imposed elsewhere
            for layer, (m, a, b) in draws.items():
                out["shake_%d_%d_mask" % (it, layer)] = m
                out["shake_%d_%d_alpha" % (it, layer)] = a
                out["shake_%d_%d_beta" % (it, layer)] = b
        arrays = {k: (np.asarray(v, np.int64) if k in ("index_map", "sizes") else np.asarray(v, np.float64 if k.startswith("loss") or k == "input_checksum" else np.float32))
                  for k, v in out.items()}
        path = os.path.join(ROOT, "tests", "golden", name + ".npz")
        np.savez_compressed(path, **arrays)
        print("%-32s P=%-7d %6.1f KiB" % (name, out["sizes"][0], os.path.getsize(path) / 1024.0))


if __name__ == "__main__":
    main()
