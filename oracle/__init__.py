"""CPU restatement of the reference's projection / MLP path.

TEST INFRASTRUCTURE ONLY. Nothing under this directory is part of the product: it is
imported by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs as the
checker (or as the timed CPU baseline), never by causal_tuner_b200 itself.

Each function restates one piece of RealJosephus/causal-tuner and cites the file:line it
follows. Pinning: tests/test_oracle_golden.py checks every function here against fixtures
in tests/golden/ that were produced by running the reference's own code in a container
where it is importable (tests/golden/make_golden.py is the generating script):
  * the NF4 decode against the reference's Triton kernel executed by the Triton interpreter
    with fp32 storage (the interpreter's bf16 conversion truncates, the GPU's rounds to
    nearest even, so 16-bit outputs are pinned as round-to-nearest-even of the fp32 golden);
  * projection, SwiGLU MLP and RoPE against the reference's CPU branch
    (modeling/lora.py:29-39, modeling/model.py:127-131, modeling/rotary.py:16-24) and
    torch autograd.
NF4 *encoding* lives in bitsandbytes, which the reference does not vendor: parity unpinned
for the encoder. Both sides of every test decode the same packed bytes, so the encoder
cannot affect a parity result.
"""
