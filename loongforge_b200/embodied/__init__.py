"""Torch-native training and evaluation stack for embodied (vision-language-action / world-model) policies.

Separate from the Megatron-style LLM stack: models are plain ``nn.Module``s wrapped in DDP, ZeRO-1 or FSDP2;
counterpart of the reference's ``loongforge/embodied`` package (entry ``train.py``, trainers, distributed
wrappers, checkpointing, optimizer adapters, datasets, policies and the evaluation framework).
"""
