"""churten_b200: the fused batched optimizer step of torchstrap, native to B200 (sm_100a).

Sub-packages mirror the reference's layout for the one path this library covers:

    churten_b200.kernels     torch.ops.torchstrap.{adam,sgd,adagrad}_step_  (CUDA key)
    churten_b200.state       State: consolidated (N, T) params / grads / optimizer state
    churten_b200.optimizer   Adam, SGD, Adagrad front-ends (init / update / apply_gradient)
    churten_b200.sharded     replica-block sharding over the GPUs of one node

Nothing is imported eagerly: `import churten_b200` works without the CUDA library,
`import churten_b200.kernels` (and everything that steps) does not.
"""

__version__ = "0.3.0"
