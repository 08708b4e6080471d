"""One rank of a sharded engine, run as a child process by test_gpu_multi.py:
python -m tests.multi_worker RANK WORLD SHAPE MIX OUT_DIR [FLAGS [MODE]]

Builds this rank's shard of the seeded synthetic model, joins the communicator (the id travels
through a file in OUT_DIR), ingests a prompt, decodes greedily and writes what it saw."""
import os
import sys
import time

import numpy as np

SEED, N_PROMPT, N_DECODE = 4242, 12, 16


def prompt(vocab: int, s: int) -> np.ndarray:
    return np.random.default_rng(SEED + s).integers(0, vocab, N_PROMPT).astype(np.int32)


def run_model(eng, cfg):
    """The same calls on a sharded rank and on the single-GPU engine it is compared with."""
    firsts = [eng.prefill_tokens(s, prompt(cfg.vocab, s), 0) for s in range(2)]
    # a probe step with fixed tokens (the same inputs whatever the greedy streams do); its KV rows are
    # rewritten by the decode below
    _, probe_logits, probe_hidden = eng.step_batch([0, 1], [5, 9], [N_PROMPT] * 2, want_logits=True, want_hidden=True)
    toks = eng.decode_greedy([0, 1], firsts, [N_PROMPT, N_PROMPT], N_DECODE)
    # one more step at the next position, with logits and hidden rows read back
    last = [int(t) for t in toks[-1]]
    nxt, logits, hidden = eng.step_batch([0, 1], last, [N_PROMPT + N_DECODE] * 2, want_logits=True, want_hidden=True)
    return dict(firsts=np.array(firsts), tokens=toks, next=nxt, logits=logits, hidden=hidden, probe_logits=probe_logits,
                probe_hidden=probe_hidden)


def main():
    rank, world, shape, mix, out_dir = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5]
    flags = int(sys.argv[6]) if len(sys.argv) > 6 else 0
    mode = sys.argv[7] if len(sys.argv) > 7 else "run"
    import camelid_b200 as cm
    from camelid_b200 import ResidentDecode, shard, synth
    from camelid_b200._lib import check, lib

    check(lib().cmld_set_device(rank))  # weights are made on the current device

    cfg = shard.rank_config(synth.engine_config(shape, max_pos=64, max_seqs=2, device=rank, flags=flags), rank, world)
    eng = synth.build_engine(cfg, mix, SEED)
    id_path = os.path.join(out_dir, "comm_id.bin")
    if rank == 0:
        with open(id_path + ".tmp", "wb") as f:
            f.write(ResidentDecode.comm_unique_id())
        os.replace(id_path + ".tmp", id_path)
    deadline = time.time() + 120
    while not os.path.exists(id_path):
        if time.time() > deadline:
            raise SystemExit("rank 0 never published the communicator id")
        time.sleep(0.05)
    with open(id_path, "rb") as f:
        uid = f.read()
    eng.comm_init(uid, rank, world)
    if mode == "run":
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), **run_model(eng, cfg))
    else:
        import faulthandler

        faulthandler.dump_traceback_later(70, exit=True)  # a stuck teardown must show where, and end
        # "leave": every rank but 0 goes away between steps, with nothing of its own in flight; rank 0
        # takes one more step, which must end in a timeout error and not in a hang
        first = eng.prefill_tokens(0, prompt(cfg.vocab, 0), 0)
        eng.decode_greedy([0], [first], [N_PROMPT], 4)
        if rank != 0:
            eng.close()
            return
        time.sleep(1.0)
        t0 = time.time()
        try:
            eng.decode_greedy([0], [first], [N_PROMPT + 4], 2)
            outcome = "no error"
        except cm.CmldError as err:
            outcome = f"code={err.code}"
        waited = time.time() - t0
        try:
            eng.decode_greedy([0], [first], [N_PROMPT + 4], 1)
            after = "no error"
        except cm.CmldError as err:
            after = f"code={err.code}"
        with open(os.path.join(out_dir, "leave.txt"), "w") as f:
            f.write(f"{outcome} {after} {waited:.2f}\n")
    eng.close()


if __name__ == "__main__":
    main()
