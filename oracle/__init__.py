"""CPU oracle for the token-sparse attention hot path.

TEST INFRASTRUCTURE ONLY.  These are plain PyTorch CPU (fp32 / fp64) restatements
of the reference's algorithms, used as the checker by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference`` legs
of ``bench.py``.  Nothing in the shipped package (``mcsparse_b200``) imports this.

Pinning status (how each restatement is anchored to the reference):

* gather-KV attention (``gather_attn``): the reference has no CPU implementation of
  this operator and no numerical test, golden vector or known-answer test for it; its
  CUDA kernels are Hopper-only and cannot run here.  PARITY UNPINNED against
  reference outputs; the restatement follows the documented contract
  (interface.py:121-136, flash_fwd_sm90.py:826-829, softmax.py:126-227) and is
  cross-checked against dense torch attention on full index sets
  (``tests/test_oracle.py``).
* group mass (``group_mass``): pinned — restates block_probs.py:27-89 and is compared with
  outputs of that very Triton kernel, executed on the CPU by Triton's interpreter on
  seeded fp16 and bf16-valued inputs (``tests/golden/mass_reference.pt``, written by
  ``tests/golden/make_golden.py``); also cross-checked against the identity
  sum_j tp = 1.
* token selection (``select``): pinned — compared on CPU with the reference's own
  ``_select_topk_tokens`` imported from the reference tree when it is present, and
  with committed golden vectors generated from it (``tests/golden``).
* Fast PDDP (``pddp``): pinned — compared on CPU with the reference's own
  ``pca_group_perm`` (fp32 inputs: identical permutation) and with committed golden
  vectors generated from it.
"""
