"""`python -m apxinf_b200.serve`: the websocket policy server over one GPU.

  python -m apxinf_b200.serve --random --precision fp8 --port 8000        # random weights, latency only
  python -m apxinf_b200.serve --model-dir /path/to/pi05_libero --action-dim 7

Unmodified OpenPI websocket clients connect to it (see apxinf_b200/serving.py for the protocol).
"""
from __future__ import annotations

import argparse

from . import apxinf_py
from .serving import Pi05Policy, WebsocketPolicyServer


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__.splitlines()[0])
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--random", action="store_true", help="random weights and synthetic processors")
    source.add_argument("--model-dir", help="checkpoint directory (model.safetensors, config.json, "
                                            "norm_stats.json, tokenizer.model, calibration.json, tactics.json)")
    parser.add_argument("--host", default="0.0.0.0")
    parser.add_argument("--port", type=int, default=8000)
    parser.add_argument("--device", default="cuda:0")
    parser.add_argument("--precision", default=None, help="bf16 | fp8 | int8 (| auto with --model-dir)")
    parser.add_argument("--calibration", default=None, help="uniform:<scale> (random) or a calibration json")
    parser.add_argument("--tactics", default=None)
    parser.add_argument("--views", type=int, default=2)
    parser.add_argument("--action-horizon", type=int, default=None)
    parser.add_argument("--action-dim", type=int, default=None, help="trim the action vector to the task's width")
    parser.add_argument("--token-count", type=int, default=10, help="synthetic prompt length (--random)")
    parser.add_argument("--discrete-state", action="store_true")
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args(argv)
    if args.random:
        precision = args.precision or "fp8"
        calibration = args.calibration or ("uniform:0.05" if precision == "fp8" else None)
        model = apxinf_py.Model.random("pi05", device=args.device, precision=precision, num_views=args.views,
                                       action_horizon=args.action_horizon or 10, calibration=calibration,
                                       seed=args.seed)
        policy = Pi05Policy.from_random(model, token_count=args.token_count, action_dim=args.action_dim,
                                        seed=args.seed)
    else:
        policy = Pi05Policy.from_pretrained(args.model_dir, device=args.device, precision=args.precision or "auto",
                                            calibration=args.calibration, tactics=args.tactics,
                                            action_dim=args.action_dim, action_horizon=args.action_horizon,
                                            seed=args.seed, discrete_state=args.discrete_state)
    print(f"serving {policy.metadata} on {args.host}:{args.port}", flush=True)
    WebsocketPolicyServer(policy, args.host, args.port).serve_forever()


if __name__ == "__main__":
    main()
