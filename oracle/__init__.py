"""CPU oracle of the hot path: TEST INFRASTRUCTURE, never imported by the product.

llama_cpu.py restates, with torch CPU arithmetic (the arithmetic of DIPU's forced CPU fallback), the decoder layer and
its single ops; it is pinned by the fixtures in tests/golden/, which were produced by the reference's own Python model.
"""
