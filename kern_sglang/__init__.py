"""SGLang plugin: the same hosted-manifest contract over SGLang's memory pools (token-to-KV pool, per-request state
pools for recurrent layers). Reference counterpart: crates/kern-py/python/kern_sglang/model.py:1-312."""
