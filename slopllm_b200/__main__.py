"""`python -m slopllm_b200 <command> ...` dispatches to the entry points in `slopllm_b200.cli`
(reference: `src/main.ts`)."""
import sys

COMMANDS = {
    "serve": "slopllm_b200.cli.serve",
    "chat": "slopllm_b200.cli.chat",
    "prefill-bench": "slopllm_b200.cli.prefill_bench",
    "sweep": "slopllm_b200.cli.sweep",
    "nll": "slopllm_b200.cli.nll",
    "mtp-bench": "slopllm_b200.cli.mtp_bench",
    "loader": "slopllm_b200.cli.model_loader",
    "weights-doc": "slopllm_b200.cli.weights_doc",
    "plan": "slopllm_b200.cli.plan",
    "kernel-bench": "slopllm_b200.cli.kernel_bench",
    "profile-step": "slopllm_b200.cli.profile_step",
    "collective-bench": "slopllm_b200.cli.collective_bench",
    "build": "slopllm_b200.build_native",
}


def main() -> int:
    if len(sys.argv) < 2 or sys.argv[1] not in COMMANDS:
        print("usage: python -m slopllm_b200 {" + ",".join(COMMANDS) + "} [options]", file=sys.stderr)
        return 2
    import importlib
    mod = importlib.import_module(COMMANDS[sys.argv[1]])
    sys.argv = [COMMANDS[sys.argv[1]]] + sys.argv[2:]
    return int(mod.main() or 0)


if __name__ == "__main__":
    raise SystemExit(main())
