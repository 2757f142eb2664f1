"""Generates tests/golden/checkpoint/<case>.nn.gz and <case>.net: the files the UNMODIFIED reference's
Save_Dimension_Parameters / Save_General_Parameters (Neural_Network__Save.cpp:204, :23) write for a case of
tests/cases.py after its two training steps, i.e. for the very state whose parameters and running normalization
statistics tests/golden/<case>.npz holds ("param1", "norm_mean_avg", "norm_sigma_avg").  Run from the repository root:

    python tests/golden/make_checkpoint_golden.py [case ...]

Needs oracle/_ref/libmyea_ref.so (oracle/build_ref.sh).
"""
import gzip
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import cases  # noqa: E402
from oracle import ref  # noqa: E402

DEFAULT = ["mlp_brn_elu_adabound_wd", "mlp_tanh_nesterov_ce", "lstm2_zoneout_clip", "res_bn_tanh_adam_noshake"]


def main():
    out_dir = os.path.join(ROOT, "tests", "golden", "checkpoint")
    os.makedirs(out_dir, exist_ok=True)
    for name in sys.argv[1:] or DEFAULT:
        wl = cases.CASES[name]()
        net = ref.RefNet(wl.desc, wl.opt, threads=1)
        cases.run_steps(net, wl)
        nn, general = os.path.join(out_dir, name + ".nn"), os.path.join(out_dir, name + ".net")
        net.save(nn, general)
        net.close()
        with open(nn, "rb") as f, gzip.GzipFile(nn + ".gz", "wb", mtime=0) as g:
            g.write(f.read())
        os.remove(nn)
        print("%-32s %6.1f KiB" % (name, os.path.getsize(nn + ".gz") / 1024.0))


if __name__ == "__main__":
    main()
