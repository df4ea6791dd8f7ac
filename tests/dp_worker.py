"""Worker for the multi-rank tests (launched with torch.distributed.run, one process per rank).

mode "cpu": world_size gloo ranks on CPU.  Each rank takes its slice of a seeded global batch, computes
  loss and gradients with the CPU checker, and the ranks average them (the CPU model of the engine's
  NCCL exchange).  Rank 0 checks that the result equals the checker run on the whole batch, i.e. that
  batch sharding + gradient averaging is exactly the single-device step.
mode "leave" / "vanish": three gloo ranks on CPU run steps with a gradient all-reduce; after step 1 the last rank leaves --
  announcing it at the step boundary ("leave") or exiting without a word ("vanish").  The others must learn of it on the
  host before their next collective (Membership.agree), rebuild a two-rank group and finish the remaining steps with
  averages taken over the survivors only; nobody may block in a collective that the departed rank never joins.
mode "gpu": one rank per GPU.  Each rank runs the device-resident engine on its slice with the NCCL
  gradient exchange enabled, then one AdamW step; rank 0 compares gradients, loss and updated weights
  with a single-device run of the engine on the whole batch.
Writes "OK" or the failure to the file given as argv[2].
"""
import importlib
import os
import sys
import traceback

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
synth = importlib.import_module("large-language-model_b200.synth")
dp = importlib.import_module("large-language-model_b200.dp")


def rel(a, b):
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    return float(np.linalg.norm(a - b) / (np.linalg.norm(b) + 1e-30))


def main():
    mode, out_path = sys.argv[1], sys.argv[2]
    from oracle import oracle
    rank, world = dp.init_control_plane("gloo")
    msg = "OK"
    try:
        per = 2
        cfg_all = oracle.Config(B=per * world, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=128, L=2)
        cfg_one = oracle.Config(B=per, S=16, H=64, I=96, nH=4, nKV=2, hd=16, V=128, L=2)
        params = synth.model_params(5, cfg_all)
        tok = synth.token_ids(5, "tokens", (cfg_all.B, cfg_all.S + 1), cfg_all.V)
        mine = dp.shard_batch(tok, rank, world)
        t, y = np.ascontiguousarray(mine[:, :-1]), np.ascontiguousarray(mine[:, 1:])
        ta, ya = np.ascontiguousarray(tok[:, :-1]), np.ascontiguousarray(tok[:, 1:])
        payload = dp.broadcast_bytes(b"id-from-rank-0" if rank == 0 else None)
        assert payload == b"id-from-rank-0"
        assert dp.max_over_ranks([float(rank)])[0] == float(world - 1)
        if mode in ("leave", "vanish"):
            import datetime
            import torch
            import torch.distributed as dist
            store = dist.TCPStore("127.0.0.1", int(os.environ["MASTER_PORT"]) + 1, world, is_master=(rank == 0),
                                  timeout=datetime.timedelta(seconds=30))
            mem = dp.Membership(store, rank, world, timeout_s=3.0)
            group, members = None, list(range(world))       # None = the default (all ranks) group
            leaver = world - 1
            for step in range(4):
                going = rank == leaver and step == 2        # departs at the boundary before step 2
                if going and mode == "vanish":
                    os._exit(0)                             # no announcement, no clean-up: the others must time out on it
                live = mem.agree(step, leaving=going)
                if going:
                    break
                if live != members:                         # somebody left: a new group over the survivors, made by them alone
                    assert leaver not in live and rank in live, (live, rank)
                    members = live
                    # creation is collective over the survivors only; the departed rank cannot take part
                    group = dist.new_group(ranks=members, use_local_synchronization=True)
                g = torch.full((4,), float(rank + 1) * (step + 1), dtype=torch.float64)
                dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
                g /= len(members)
                expect = np.mean([float(r + 1) * (step + 1) for r in members])
                assert abs(float(g[0]) - expect) < 1e-12, (step, members, float(g[0]), expect)
            if rank != leaver:
                assert members == [r for r in range(world) if r != leaver], members
            with open(out_path + f".rank{rank}", "w") as f:
                f.write("OK")
            os._exit(0)     # the default group still counts the departed rank: no collective tear-down with it
        if mode == "cpu":
            orc = oracle.Oracle()
            loss, grads, _ = orc.model_loss_and_grads(cfg_one, t, y, params)
            g_avg = dp.average_over_ranks(grads)
            l_avg = dp.average_over_ranks(np.array([loss]))[0]
            if rank == 0:
                loss_all, grads_all, _ = orc.model_loss_and_grads(cfg_all, ta, ya, params)
                assert abs(l_avg - loss_all) < 1e-5, (l_avg, loss_all)
                assert rel(g_avg, grads_all) < 1e-5, rel(g_avg, grads_all)
        else:
            import torch
            bridge = importlib.import_module("large-language-model_b200.bridge")
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            ctx = bridge.Context(local)
            model = bridge.Model(ctx, cfg_one, "f32")
            model.load_params(params)
            uid = dp.broadcast_bytes(bridge.dp_unique_id() if rank == 0 else None)
            model.dp_init(uid, rank, world)
            loss = model.loss_and_grads_host(t, y)
            grads = model.read_grads()
            model.adamw_step(1e-2)
            new_params = model.read_params()
            l_avg = dp.average_over_ranks(np.array([loss]))[0]
            model.close()
            # whole training steps: the optimizer is sharded over the ranks (reduce-scatter, AdamW on one slice per rank,
            # all-gather of the weights); reading the weights back gathers the fp32 masters from all ranks
            stepper = bridge.Model(ctx, cfg_one, "f32")
            stepper.load_params(params)
            uid2 = dp.broadcast_bytes(bridge.dp_unique_id() if rank == 0 else None)
            stepper.dp_init(uid2, rank, world)
            step_losses = [stepper.train_step_host(t, y, lr=1e-2) for _ in range(3)]
            stepped = stepper.read_params()
            m_sh, v_sh, n_sh = stepper.read_opt_state()
            stepper.close(); ctx.close()
            step_l_avg = [dp.average_over_ranks(np.array([l]))[0] for l in step_losses]
            if rank == 0:
                ctx1 = bridge.Context(local)
                single = bridge.Model(ctx1, cfg_all, "f32")
                single.load_params(params)
                loss_all = single.loss_and_grads_host(ta, ya)
                grads_all = single.read_grads()
                single.adamw_step(1e-2)
                params_all = single.read_params()
                single.close()
                one = bridge.Model(ctx1, cfg_all, "f32")
                one.load_params(params)
                one_losses = [one.train_step_host(ta, ya, lr=1e-2) for _ in range(3)]
                one_params = one.read_params()
                m_one, v_one, n_one = one.read_opt_state()
                one.close(); ctx1.close()
                assert np.allclose(step_l_avg, one_losses, rtol=1e-5, atol=1e-6), (step_l_avg, one_losses)
                assert rel(stepped, one_params) < 1e-5, rel(stepped, one_params)
                assert n_sh == n_one == 3 and rel(m_sh, m_one) < 1e-4 and rel(v_sh, v_one) < 1e-4
                assert abs(l_avg - loss_all) < 1e-5, (l_avg, loss_all)
                assert rel(grads, grads_all) < 1e-4, rel(grads, grads_all)
                assert rel(new_params, params_all) < 1e-5, rel(new_params, params_all)
    except Exception:      # noqa: BLE001 - reported to the parent test
        msg = traceback.format_exc()
    import torch.distributed as dist
    flags = [None] * world
    if dist.is_initialized():
        dist.all_gather_object(flags, msg)
    else:
        flags = [msg]
    if rank == 0:
        bad = [m for m in flags if m != "OK"]
        with open(out_path, "w") as f:
            f.write("OK" if not bad else "\n".join(bad))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
