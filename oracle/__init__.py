"""CPU oracle for the decode-attention path.  TEST INFRASTRUCTURE ONLY.

``cpu_oracle`` wraps the C restatement (``sa_oracle.c``, double accumulation);
``torch_port`` restates the reference's own CPU PyTorch path and is what the
benchmark times as the CPU baseline.  Only tests, the smoke check and the
benchmark's CPU-baseline leg may import this package; the shipped
``streamattn_b200`` package never does.

Parity status: pinned against outputs of the reference itself and against the
reference's own test vectors (fixtures and generator under ``tests/golden/``).
"""
