"""system_lab_b200 — a Blackwell (sm_100a) native MoE training framework.

Layers (top to bottom):

* ``train`` / ``pilot``  — command line entry points (trainer, tuning agent)
* ``config``             — typed configuration in Megatron knob vocabulary
* ``trainer``            — step loop, optimizer, LR schedule, metrics, events
* ``parallel``           — device mesh, FSDP engine, expert/pipeline/context parallel
* ``models``             — SimpleMoE decoder family (GQA and MLA attention)
* ``moe``                — router, dispatch/combine, grouped experts
* ``comm``               — symmetric peer memory, flag protocol, NCCL baseline
* ``ops`` + ``csrc``     — hand written sm_100a kernels and their PyTorch oracles
* ``ckpt``               — sharded, reshardable checkpoints
* ``observe``            — profiler hooks, Kineto trace breakdown, roofline reports
"""

__version__ = "0.1.0"
