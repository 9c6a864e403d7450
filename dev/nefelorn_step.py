"""Run prefill or single-token steps of a random-weight Nefelorn (or, ``--model salizen`` / ``--model zubarax``, Salizen / Zubarax) model of one of the
serving-bench sizes — a small, one-model workload for a profiler (launch lists, captures of one kernel):

    python dev/nefelorn_step.py --size w2048 --phase prefill --batch 8 --prompt 2048 --iters 2 [--model salizen]
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

import torch  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", choices=["nefelorn", "salizen", "zubarax"], default="nefelorn")
    ap.add_argument("--size", default="w1024")
    ap.add_argument("--phase", choices=["prefill", "decode"], default="prefill")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=2)
    ap.add_argument("--graphs", type=int, default=0)
    a = ap.parse_args()
    from libai_b200 import ops
    from libai_b200.config import DictConfig
    from libai_b200.inference import serving_bench as sb
    from libai_b200.inference.scheduler import RequestScheduler
    from libai_b200.layers._param import param_defaults
    from libai_b200.models import NefelornForCausalLM, SalizenForCausalLM, ZubaraxForCausalLM

    s = sb.NEFELORN_SIZES[a.size]
    with param_defaults(dtype=torch.bfloat16, device="cuda", seed=1):
        if a.model == "zubarax":
            model = ZubaraxForCausalLM(DictConfig(sb.zubarax_config(s))).eval().cuda()
        elif a.model == "salizen":
            model = SalizenForCausalLM(DictConfig(sb.salizen_config(s))).eval().cuda()
        else:
            model = NefelornForCausalLM(DictConfig(sb.nefelorn_config(s))).eval().cuda()
    sched = RequestScheduler(model, cuda_graphs=bool(a.graphs))
    ids = torch.randint(1, s["vocab"], (a.batch, a.prompt), generator=torch.Generator().manual_seed(0))
    prompts = [row.tolist() for row in ids]
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if a.phase == "prefill":
        for it in range(a.iters):
            ops.reset_launch_count()
            ev0.record()
            sched.step([(("p", i), p, [len(p) - 1]) for i, p in enumerate(prompts)])
            ev1.record()
            sched.finish([("p", i) for i in range(a.batch)])
            torch.cuda.synchronize()
            print(f"prefill {it}: {ev0.elapsed_time(ev1):.3f} ms, {ops.launch_count()} launches", flush=True)
    else:
        sched.step([(("d", i), p, []) for i, p in enumerate(prompts)])
        for it in range(a.iters):
            ops.reset_launch_count()
            ev0.record()
            sched.step([(("d", i), [7], [0]) for i in range(a.batch)])
            ev1.record()
            torch.cuda.synchronize()
            print(f"decode {it}: {ev0.elapsed_time(ev1):.3f} ms, {ops.launch_count()} launches", flush=True)


if __name__ == "__main__":
    main()
