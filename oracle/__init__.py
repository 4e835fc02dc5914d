"""CPU oracle of the attention path (decode and prompt phase).  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs
of ``bench.py`` may import this package; nothing under ``muxserve_b200/`` does.

Pinning status
--------------
* allocator (``KVStorage``) and step builder (``BatchScheduler``): PINNED.  The
  reference's own ``csrc/memory_manager.cpp`` and ``csrc/batch_scheduler.cpp``
  compile CPU-only (``build_ref.py`` -> ``oracle/_ref/``) and are the live oracle;
  ``host_oracle.py`` restates them in Python and is checked against the compiled
  reference and against the known-answer traces under ``tests/golden/``.
* ``reshape_and_cache`` and ``paged_attention``: PARITY UNPINNED.  Their source
  lives in the third-party fork EfficientLLMSys/MuxServe-vLLM, which the reference
  names without a version or commit (README.md:16-25, requirements.txt:1-2) and
  which is absent here; the reference holds no test or golden vector for them.
  ``cache_write_oracle.py`` and ``attention_oracle.py`` restate the published
  algorithm (vLLM paged attention) on the pool layout the reference defines
  (muxserve/flexstore/manager.py:456-468) and the slot formula of
  csrc/batch_scheduler.h:42-67.
* rotary embedding and prompt-phase attention (``rotary_oracle.py``, ``prefill_oracle.py``):
  PARITY UNPINNED for the same reason (the prompt branch and the rotary step are inside
  the fork's ``PagedAttentionWithRoPE``); both restate the published semantics in fp32.
"""
