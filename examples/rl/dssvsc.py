"""A non-training OneRPC service: a self-play "producer" pushes episodes to a "trainer"
node over the control plane (counterpart of the reference sketch examples/rl/dssvsc.py).
Shows ``TmplServer`` / ``TmplService`` used directly: endpoints only enqueue, the service's
``check_state`` timer does the work.

    python dssvsc.py trainer  ipc:///tmp/rl-trainer.ipc
    python dssvsc.py producer ipc:///tmp/rl-producer.ipc ipc:///tmp/rl-trainer.ipc
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from necklace_b200.rpc import svctmp


class TrainerServer(svctmp.TmplServer):
    def fn_push_episode(self, msg):
        m = self.msg_unpck(msg)
        self.q_put_state(1, m["msg"]["obs"], m["msg"]["reward"], m["rank"])
        return self.msg_pck(self.mk_rpc_ret("fn_push_episode", "ok"))


class TrainerService(svctmp.TmplService):
    def __init__(self, url, n_expected=5):
        super().__init__({"url": url})
        self.svr = TrainerServer({"url": url, "rank": 0, "role": "trainer"})
        self.seen, self.n_expected, self.returns = 0, n_expected, []

    def check_state(self, *a, **k):
        state, args, _ = self.q_get_state(timeout=0.1)
        if state == 1:
            obs, reward, rank = args
            self.returns.append(float(reward))
            self.seen += 1
            print(f"trainer: episode {self.seen} from producer {rank}: obs {obs.shape}, "
                  f"return {reward:.3f}")
            if self.seen >= self.n_expected:
                self.stop()


def producer(url, trainer_url, n=5):
    svr = svctmp.TmplServer({"url": url, "rank": 1, "role": "producer"})
    cli = svr.mk_rpc_cli(trainer_url)
    rng = np.random.default_rng(0)
    for _ in range(n):
        obs = rng.normal(size=(16, 8)).astype(np.float32)
        rep = svr.do_rpc_call(cli, "fn_push_episode", obs=obs, reward=float(obs.sum()))
        assert rep["ret"] == "ok"
    cli.close()
    svr.stop()


if __name__ == "__main__":
    if sys.argv[1] == "trainer":
        svc = TrainerService(sys.argv[2])
        svc.loop()
    else:
        producer(sys.argv[2], sys.argv[3])
