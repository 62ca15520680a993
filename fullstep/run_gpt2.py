"""Whole data-parallel GPT-2 training steps through the UNMODIFIED Soliton Python package and example trainer
(compiled into fullstep/_ref/ by fullstep/build.py) on top of this repository's library: forward and backward run on
the reference's own CUDA backend, the gradient mean + AdamW on this library's fused kernels.

Follows the reference's own measurement (bench/soliton_gpt2.py:57-103): plan the run on the meta device (an arena of
fixed offsets), install it, run `steps` steps of examples/gpt2.py's `run`, drop the first two from the timing, and
compare the planned bytes with the pool's peak. Tokens are uniform over the vocabulary, seeded by rank (the
reference trains on TinyStories, which is not available offline).

    python fullstep/run_gpt2.py --config 124M --batch 8 --steps 8 [--tf32] [--nproc N] [--hash]
    python fullstep/run_gpt2.py --config medium --batch 4 --steps 10 --nproc 8 --budget-gib 40 --hash

One JSON line ("FULLSTEP {...}") from rank 0: tokens/s over all ranks, step time, planned and real peak bytes, and
with --hash the SHA-256 of all parameters per rank after the last step.
"""
import argparse
import hashlib
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
REF = os.path.join(HERE, "_ref")
sys.path[:0] = [REF, ROOT]
from fullstep.build import ensure_importable  # noqa: E402
ensure_importable()

V = 50257


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="124M", choices=["124M", "medium", "tiny"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--tf32", action="store_true")
    ap.add_argument("--no-arena", action="store_true")
    ap.add_argument("--budget-gib", type=float, default=0.0, help="solve recomputation so that the step fits this budget")
    ap.add_argument("--nproc", type=int, default=1)
    ap.add_argument("--hash", action="store_true")
    ap.add_argument("--dp", default="ours", choices=["ours", "reference"],
                    help="reference: gradient mean and AdamW on the reference's own NCCL + k_adamw instead of this library")
    ap.add_argument("--timeout", type=float, default=1500.0)
    args = ap.parse_args()

    os.environ["SOLITON_FULLSTEP_DP"] = args.dp
    if args.nproc > 1 and "RANK" not in os.environ:
        from soliton_b200.launch import launch_workers
        sys.exit(launch_workers(args.nproc, [sys.executable, os.path.abspath(__file__), *sys.argv[1:]], timeout=args.timeout))

    import numpy as np
    import gpt2                      # the reference's example, unmodified
    import soliton as sl             # the reference's package, unmodified, bound to fullstep/_ref/soliton/libsoliton.so
    from soliton import distributed

    # GPT-2 medium is not among the example's configurations (examples/gpt2.py:76-79): same layout, more of it
    gpt2.CONFIGS.setdefault("medium", dict(n_layer=24, n_head=16, n_embd=1024))
    vocab = gpt2.CONFIGS[args.config].get("vocab", V)
    seq = min(args.seq, gpt2.CONFIGS[args.config].get("block_size", 1024))
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))

    t0 = time.time()
    ckpt = 0
    if args.budget_gib:
        ckpt, _ = gpt2.fit_checkpoints(args.config, args.batch, seq, 1, int(args.budget_gib * 2**30))
        if ckpt is None:
            sys.exit("does not fit the budget even with everything recomputed")
    plan = None
    if not args.no_arena:
        plan = sl.arena.plan(lambda d: gpt2.run(d, args.config, args.batch, seq, 1, 2, checkpoint=ckpt))
        predicted = plan.bytes
    else:
        predicted = sl.plan(lambda d: gpt2.run(d, args.config, args.batch, seq, 1, 2, checkpoint=ckpt))["peak_reserved"]
    plan_s = time.time() - t0

    if world > 1:
        distributed.init(rank, world, os.environ["SOLITON_INIT_FILE"])
    else:
        sl.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if args.tf32:
        sl.set_tf32(True)
    base_reserved = sl.memory_stats("cuda")["reserved"]      # device initialisation's fixed workspaces
    if plan is not None:
        sl.arena.install(plan, "cuda")

    rng = np.random.default_rng(rank)                        # each rank sees different batches

    def get_batch():
        tok = rng.integers(0, vocab, size=(args.batch, seq + 1)).astype(np.int32)
        return tok[:, :-1], tok[:, 1:]

    times = []
    stats, losses, model, opt = gpt2.run("cuda", args.config, args.batch, seq, 1, args.steps, get_batch,
                                         log=lambda step, loss, norm, dt: times.append(dt), checkpoint=ckpt)
    if plan is not None:
        sl.arena.check("cuda")
    digest = None
    if args.hash:
        h = hashlib.sha256()
        for p in model.parameters():
            h.update(p.numpy().tobytes())
        digest = h.hexdigest()
    warm = times[2:] or times
    out = {"rank": rank, "world": world, "config": args.config, "batch_per_rank": args.batch, "seq": seq, "steps": args.steps,
           "matmul": "tf32" if args.tf32 else "fp32", "data_parallel_path": args.dp, "allocator": "pool" if plan is None else "arena",
           "recomputed_units": ckpt if isinstance(ckpt, int) else len(ckpt),
           "step_ms": 1000 * sum(warm) / len(warm), "tokens_per_s": args.batch * seq * world * len(warm) / sum(warm),
           "loss_first": losses[0], "loss_last": losses[-1], "plan_seconds": plan_s,
           "predicted_bytes": int(predicted),
           "real_bytes": int(stats["peak_reserved"] - (base_reserved if plan is not None else 0)),
           "fixed_workspaces_bytes": int(base_reserved), "sha256": digest}
    out["prediction_error_bytes"] = out["real_bytes"] - out["predicted_bytes"]

    if world > 1:   # collect every rank's line on rank 0 through files next to the group id
        d = os.path.dirname(os.environ["SOLITON_INIT_FILE"])
        with open(os.path.join(d, f"result.{rank}.tmp"), "w") as f:
            json.dump(out, f)
        os.replace(os.path.join(d, f"result.{rank}.tmp"), os.path.join(d, f"result.{rank}"))
        if rank == 0:
            deadline = time.time() + 300
            rows = []
            for r in range(world):
                path = os.path.join(d, f"result.{r}")
                while not os.path.exists(path) and time.time() < deadline:
                    time.sleep(0.05)
                rows.append(json.load(open(path)))
            out["step_ms"] = max(r["step_ms"] for r in rows)
            out["tokens_per_s"] = args.batch * seq * world / (out["step_ms"] / 1000)
            out["sha256_per_rank"] = [r["sha256"] for r in rows]
            out["bit_identical_across_ranks"] = len(set(out["sha256_per_rank"])) == 1 if args.hash else None
            out["prediction_error_bytes_per_rank"] = [r["prediction_error_bytes"] for r in rows]
    if rank == 0:
        print("FULLSTEP " + json.dumps(out), flush=True)
    sl.arena.off("cuda") if plan is not None else None


if __name__ == "__main__":
    main()
