"""CPU restatement of the AMCT quantization hot path. TEST INFRASTRUCTURE ONLY.

Nothing under ``amct_b200`` may import this package: it is the checker that the
CUDA path is compared against in ``tests/``, in ``__graft_entry__.smoke()`` and
in the CPU-baseline leg of ``bench.py``.  The product path has no CPU fallback.

Modules
-------
intq     integer quantization arithmetic the reference implements in torch
         (scale/offset, codes, fake-quant, SmoothQuant fold, deploy constants).
         PINNED: checked against outputs of the imported reference, committed
         as fixtures under ``tests/golden`` (``tests/golden/make_golden.py``).
npu_ops  the four external ``torch_npu`` ops the deploy modules call.  The
         reference does not contain them and its tests mock them without
         rounding or scaling, so this part is PARITY UNPINNED: it restates the
         documented formula and the operand construction at the call sites.
mx       MXFP8-E4M3 / MXFP4-E2M1 with E8M0 block scales.  Absent from the
         reference: PARITY UNPINNED, restated from the public OCP MX v1.0 rules.
ckpt     the offline checkpoint formats of the reference's DeepSeek-V3.2 export script (FP8 block dequant,
         per-channel INT8 / INT4 with nibble packing, uint64 scale words, INT4 assistance bias, Hadamard
         matrix).  PINNED: checked against outputs of the imported reference script, committed as
         ``tests/golden/ckpt_golden.*`` (``tests/golden/make_ckpt_golden.py``).
dsa      the KV-cache / indexer activation path of the same tree: per-token dynamic fake quantization
         (ActivationQuantizer) and the Hadamard rotation.  PINNED: checked against outputs of the imported
         reference modules, committed as ``tests/golden/dsa_golden.npz`` (``tests/golden/make_dsa_golden.py``).
hif8     HiFloat8 encode/decode.  Absent from the reference: PARITY UNPINNED,
         restated from the published format description.
"""
