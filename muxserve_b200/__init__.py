"""B200-native decode attention path for MuxServe's unified, head-granular KV pool.

Modules mirror the reference's units on this path:
``ops`` (paged_attention / reshape_and_cache), ``memory_manager`` (KVStorage),
``batch_scheduler`` (BatchScheduler), ``flexstore`` (pool geometry),
``mixed`` (descriptors for one launch over several models).
Importing the package does not load the CUDA library; the first op call does,
and fails loudly if it has not been built.
"""
__version__ = "0.1.0"
