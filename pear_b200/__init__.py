"""pear_b200: a Blackwell-native (B200, sm_100a) asynchronous RL post-training engine.

Sub-packages
------------
config    recipe/config loader with the upstream key names (YAML + dotted overrides)
models    hybrid Gated-DeltaNet + gated-attention decoder, MTP head, drafter, NVFP4, safetensors IO
ops       hand-written sm_100a CUDA kernels (csrc/) with ctypes bindings and fp32 torch references
parallel  process groups, symmetric memory / peer pointers, FSDP sharder, Ulysses SP, GDN context parallel, TP
train     GRPO trainer, engine, streamed AdamW, checkpointing, activation offload, replay buffer
rollout   paged-KV rollout engine: scheduler, prefix cache, host tier, sampler, MTP speculative decoding
loop      async agent loop, transfer queue, weight sync
sim/envs  simulator runtime (server pool, supervised processes) and the seeded synthetic environment
deploy    batch-1 NVFP4 persistent decode megakernel: instruction scheduler, runner, server
eval      embodied and general evaluation entry points
monitor   metrics scraping, progress tracker, driver log parser, progress panel
launch    role-based launcher (trainer / rollout / agent)
"""

__version__ = "0.1.0"
