"""The list of kernel objects: (source file, -D defines).  Units without defines take
every size at run time; units specialised on a head size exist once per size in
``HEAD_SIZES`` and any other size is compiled when a model first asks for it."""
from __future__ import annotations

GENERIC_UNITS = [("elementwise.cu", ()), ("gemm_simt.cu", ()), ("attn_generic.cu", ()),
                 ("sampling.cu", ()), ("random_init.cu", ())]

# head sizes built ahead of time (what the tests and the benchmark use)
HEAD_SIZES = (64, 128)

SPECIALISED_SOURCES: list = []          # filled by the bfloat16 kernels' bindings
BF16_UNITS: list = []                   # bfloat16 kernels that take every size at run time


def all_units() -> list:
    from .. import kernels_bf16  # noqa: F401  (registers the bfloat16 kernels' sources)
    units = list(GENERIC_UNITS) + [(s, ()) for s, _ in BF16_UNITS]
    for src, extra in SPECIALISED_SOURCES:
        for hd in HEAD_SIZES:
            units.append((src, (f"HD={hd}",) + tuple(extra)))
    return units


# Builds that only the tests load: the tcgen05 kernels with a short wait limit and a copy role
# that issues nothing, so that a test can see every other role give up and the kernel return.
WAITS_RUN_OUT = ("G2B_SPIN_LIMIT=4096", "G2B_TEST_NO_PRODUCER")
TEST_UNITS = [("gemm_tc.cu", WAITS_RUN_OUT), ("attn_prefill_tc.cu", ("HD=128",) + WAITS_RUN_OUT),
              ("attn_prefill_tc_split.cu", ("HD=128",) + WAITS_RUN_OUT)]
