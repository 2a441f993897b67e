"""Evaluation framework of the embodied stack: policy server, msgpack-numpy RPC, protocol schema, payload builders,
action decoders, environment adapters, orchestrator and reports (reference: loongforge/embodied/eval/*)."""
