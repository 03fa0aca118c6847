"""CPU oracle for the Point Transformer V3 inference path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: it is used by the tests, by the smoke check and by the CPU-baseline
leg of the benchmark, always as the checker or the timed CPU reference and
never as a fallback of the CUDA path.

* ``encode_oracle.c``  plain-C restatement of the serialization stage.
* ``cenc.py``          ctypes loader for that C file.
* ``ptv3_oracle.py``   torch-on-CPU restatement of the remaining stages
                       (padding plan, patch attention, submanifold convolution,
                       pooling, unpooling, blocks, whole backbone).
* ``weights.py``       deterministic, name-keyed parameter fill shared by the
                       golden-vector generator and the parity tests.
* ``refshim/``         stand-ins for the four third-party packages the
                       reference model imports, so the unmodified reference
                       file can be executed on CPU where it is available.

Parity pin: the serialization stage, the padding plan, attention, pooling,
unpooling, blocks and the whole backbone are checked against the reference's
own code executed on CPU (directly where it is present, and through the golden
vectors under ``tests/golden`` everywhere).  The submanifold convolution is a
third-party kernel (spconv, not vendored by the reference, no version pinned):
for it the pin is a dense ``conv3d`` evaluated at the active sites, and parity
with spconv itself is UNPINNED.
"""
