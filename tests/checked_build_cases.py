"""Runs the tiny models through whichever library B200EMB_LIBRARY names and records the rows:

    python tests/checked_build_cases.py <workdir> normal
    B200EMB_LIBRARY=infinity_b200/lib/libb200emb_checked.so python tests/checked_build_cases.py <workdir> checked

The second call (the build with device-side index range checks) must reproduce the first call's rows
bit for bit, must report a sequence boundary that leaves the token stream instead of reading past it,
and must leave the handle usable. Driven by test_gpu_checked_build.py; not collected by pytest itself.
"""
import pathlib
import sys

import numpy as np
import torch

ROOT = pathlib.Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from helpers import build_model  # noqa: E402
from infinity_b200 import _lib  # noqa: E402
from infinity_b200 import configs as cf  # noqa: E402
from infinity_b200._lib import B200EmbError  # noqa: E402

CASES = [("bert", {}, [40, 3, 77, 128]), ("xlmr", {}, [17, 90]), ("moe", {}, [40, 3, 77, 150, 9]),
         ("moe", {"weight_format": "mxfp8"}, [40, 3, 77, 150, 9]), ("decoder", {}, [200, 31, 64]),
         ("decoder", {"weight_format": "nvfp4"}, [200, 31])]


def main() -> None:
    work = pathlib.Path(sys.argv[1])
    mode = sys.argv[2]
    lib = _lib.load()
    assert lib.b200emb_checked_build() == (1 if mode == "checked" else 0), "wrong library variant loaded"
    for n, (arch, kw, lengths) in enumerate(CASES):
        spec = cf.tiny_spec(arch, **kw)
        d = work / f"{mode}_{n}"
        d.mkdir()
        model, _ = build_model(d, spec, 31 + n, perturb=True)
        batch = cf.random_batch(spec, lengths, 7 + n)
        rows = model.forward(batch)
        assert np.isfinite(rows).all()
        if mode == "normal":
            np.save(work / f"rows_{n}.npy", rows)
        else:
            assert np.array_equal(rows, np.load(work / f"rows_{n}.npy")), f"case {n} ({arch}): rows differ from the normal build's"
        if mode == "checked" and arch == "bert":
            # The device copy of cu_seqlens disagrees with the host's: its last boundary lies beyond the token
            # stream (but inside the 1024-token workspace, so the rows exist either way). The pooling kernel
            # must notice, pool an empty range instead, and the call must say so.
            d_ids = torch.from_numpy(batch.input_ids).cuda()
            d_ty = torch.zeros(batch.n_tokens, dtype=torch.int32, device="cuda")
            wrong = batch.cu_seqlens.copy()
            wrong[-1] = batch.n_tokens + 200
            d_out = torch.empty(batch.n_seqs, spec.out_dim, dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()

            def run(cu_dev):
                d_cu = torch.from_numpy(cu_dev).cuda()
                torch.cuda.synchronize()
                model.forward_device(d_ids.data_ptr(), d_ty.data_ptr(), d_cu.data_ptr(), batch.cu_seqlens, batch.n_tokens,
                                     d_out.data_ptr())
                torch.cuda.synchronize()
                return d_out.cpu().numpy()

            try:
                run(wrong)
            except B200EmbError as e:
                assert "device index check: code 40" in str(e), str(e)
            else:
                raise AssertionError("the out-of-range sequence boundary went unnoticed")
            assert np.array_equal(run(batch.cu_seqlens), rows)   # the status words were cleared: the next forward is clean
        model.close()
    print(f"{mode}: {len(CASES)} cases ok")


if __name__ == "__main__":
    main()
