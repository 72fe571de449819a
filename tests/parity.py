"""Measured-error bookkeeping of the GPU parity tests.

``check(out, ref, max_abs, mean_rel, what)`` computes the two figures the project's tolerance is stated in
(max-abs and mean-rel = mean|out - ref| / mean|ref| over the whole tensor), prints them (shown by
``pytest -rA`` / ``-s``), appends them to the file named by the environment variable
``MOA_B200_PARITY_LOG`` when that is set, and asserts them against the given bounds.
"""
import os

# the project's tolerance against an fp32 evaluation of the same mask, for fp16 and for the
# fp32-store mode of the bf16 kernels
MAX_ABS, MEAN_REL = 2e-3, 1e-3


def errors(out, ref):
    out, ref = out.float().cpu(), ref.float().cpu()
    max_abs = (out - ref).abs().max().item()
    mean_rel = ((out - ref).abs().mean() / ref.abs().mean().clamp_min(1e-12)).item()
    return max_abs, mean_rel


def check(out, ref, max_abs=MAX_ABS, mean_rel=MEAN_REL, what=""):
    a, r = errors(out, ref)
    test = os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0]
    line = f"{test} | {what} | max-abs {a:.3e} (bound {max_abs:.1e}) | mean-rel {r:.3e} (bound {mean_rel:.1e})"
    print("[parity] " + line)
    path = os.environ.get("MOA_B200_PARITY_LOG")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")
    assert a <= max_abs and r <= mean_rel, line
    return a, r
