"""CPU restatement of SPION's layer-wise block-sparse attention path.

TEST INFRASTRUCTURE ONLY.  Nothing here is part of the shipped product: the
package under ``spion_b200/`` never imports this module.  It is imported by
``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``, always as the checker or as the
timed CPU baseline, never as the thing being shipped.

Pinning status
--------------
* pattern discovery (``oracle.pattern``): pinned.  ``tests/golden/pattern_*.npz``
  hold block masks produced by the reference's own ``flood_fill``
  (main_conv_ff.py:35-62) driven by the reference's own driver lines
  (main_conv_ff.py:255-279) on seeded inputs; ``tests/test_oracle_pattern.py``
  checks the restatement against them bit for bit.
* element CSR (``oracle.csr``): pinned the same way against
  models/attention_blockcuda.py:31-43 executed on CPU tensors.
* dense softmax attention (``oracle.attention.dense_attention``): pinned against
  the reference's ``SoftmaxAttention`` (models/attention.py:13-38).
* block-sparse attention (``oracle.attention.sparse_attention``): the reference
  has no CPU implementation and ships no test vectors for it.  The restatement
  follows models/block_attn.cu:33-130 line by line
  (``sparse_attention_rowwise``) and is cross-checked against the dense-masked
  closed form; on a GPU box it is additionally compared with the reference's
  own CUDA file compiled into ``oracle/_ref`` (see ``oracle/build_ref.py``).
* plain-C restatement (``oracle/spion_oracle.c``, bound by ``oracle.c_oracle``, built by
  ``oracle/build_c.py``): a second, independent restatement of all three parts.
  ``tests/test_oracle_c.py`` requires it to reproduce the golden masks, the pooled map, the
  threshold and the CSR arrays bit for bit and the attention step within fp32 rounding.
"""
