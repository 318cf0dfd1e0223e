"""B200-native data-parallel transformer training framework.

Layers (each only calls downward):

* ``config``      -- model / optimizer / run configuration, presets, CLI flags, config validation
* ``data``        -- character tokenizer, sequential batcher, seeded synthetic token streams
* ``arena``       -- flat parameter / gradient / optimizer-state arenas in backward-production order
* ``checkpoint``  -- flat dump format, parameter statistics and FNV-1a hash (trajectory tracing)
* ``models``      -- pure-PyTorch oracle model and the native sm_100a engine
* ``ops``         -- hand-written sm_100a kernels behind a C ABI, loaded with ctypes
* ``parallel``    -- data-parallel gradient synchronisation (blocking, bucketed overlap, fused peer-memory)
* ``utils``       -- device timers, NVTX ranges, clock sampling, log-line formats
* ``train``       -- the command-line training driver
"""

__version__ = "0.1.0"
