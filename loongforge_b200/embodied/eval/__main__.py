"""Command line of the embodied evaluation stack (reference: loongforge/embodied/eval entry scripts).

    python -m loongforge_b200.embodied.eval serve --config recipe.yaml [--checkpoint DIR] [--port P] [key=value ...]
        loads the policy of a training recipe (weights from the newest checkpoint under DIR) and serves
        ``predict_action`` over the msgpack RPC transport until interrupted
    python -m loongforge_b200.embodied.eval mock [--port P] [--horizon H] [--action-dim A]
        serves the constant mock policy (protocol smoke tests)
    python -m loongforge_b200.embodied.eval run --port P [--env reach] [--episodes N] [--output-dir DIR]
        drives an environment against a running server and writes ``report.json``
"""
from __future__ import annotations

import argparse
import json
import sys
import time


def _serve_forever(srv) -> int:
    print(json.dumps({"serving": True, "host": srv.host, "port": srv.port}), flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        pass
    finally:
        srv.stop()
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("loongforge_b200.embodied.eval")
    sub = ap.add_subparsers(dest="cmd", required=True)
    s = sub.add_parser("serve")
    s.add_argument("--config", default=None)
    s.add_argument("--checkpoint", default=None)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=0)
    s.add_argument("--denoise-steps", type=int, default=10)
    s.add_argument("--action-space", default="joint")
    s.add_argument("--once", action="store_true", help="start, print the address, stop (for tests)")
    s.add_argument("overrides", nargs="*")
    m = sub.add_parser("mock")
    m.add_argument("--host", default="127.0.0.1")
    m.add_argument("--port", type=int, default=0)
    m.add_argument("--horizon", type=int, default=8)
    m.add_argument("--action-dim", type=int, default=7)
    m.add_argument("--once", action="store_true")
    r = sub.add_parser("run")
    r.add_argument("--host", default="127.0.0.1")
    r.add_argument("--port", type=int, required=True)
    r.add_argument("--env", default="reach")
    r.add_argument("--episodes", type=int, default=10)
    r.add_argument("--output-dir", default=None)
    r.add_argument("--max-steps", type=int, default=None)
    a = ap.parse_args(argv)

    from .policy_server import MockPolicyService, PolicyService, serve
    if a.cmd == "mock":
        srv = serve(MockPolicyService(horizon=a.horizon, action_dim=a.action_dim), a.host, a.port)
        if a.once:
            print(json.dumps({"serving": True, "port": srv.port}), flush=True)
            srv.stop()
            return 0
        return _serve_forever(srv)
    if a.cmd == "serve":
        import torch

        from .. import checkpoint as ckpt
        from ..config import parse_args
        from ..models import build_policy
        args = parse_args((["--config", a.config] if a.config else []) + list(a.overrides))
        policy = build_policy(args.model_name, args)
        if a.checkpoint:
            if ckpt.load_checkpoint(a.checkpoint, policy, restore_rng=False) is None:
                raise FileNotFoundError(f"no checkpoint under {a.checkpoint}")
        policy.eval()
        if torch.cuda.is_available():
            policy.cuda()
        srv = serve(PolicyService.from_output_dir(policy, args, action_space=a.action_space, denoise_steps=a.denoise_steps), a.host, a.port)
        if a.once:
            print(json.dumps({"serving": True, "port": srv.port, "model": args.model_name}), flush=True)
            srv.stop()
            return 0
        return _serve_forever(srv)
    from .orchestrator import EvalConfig, run_evaluation
    kw = {"max_steps": a.max_steps} if a.max_steps else {}
    rep = run_evaluation(EvalConfig(env=a.env, episodes=a.episodes, host=a.host, port=a.port, output_dir=a.output_dir,
                                    env_kwargs=kw))
    print(json.dumps({k: rep[k] for k in ("success_rate", "mean_steps") if k in rep}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
