"""fastgen_b200: a single-GPU (sm_100a) inference engine for dense GQA decoders.

The package is layered bottom-up:

* ``config``   -- typed model description parsed from ``config.json`` and the
                  architecture registry.
* ``weights``  -- safetensors loading by tensor name and the random-weights
                  writer.
* ``parts``    -- mixers, feed-forwards, norms, position encodings and blocks.
* ``cache``    -- paged KV pools, block tables and fixed-size state slots.
* ``engine``   -- the step function, the scheduler and the generator API.
* ``sampling`` -- greedy / temperature / top-p sampling.
* ``csrc``     -- the CUDA sources and their in-tree builder.
"""

__version__ = "0.1.0"
