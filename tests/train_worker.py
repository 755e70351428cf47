"""Child process of test_training_cpu.py: one data-parallel rank on CPU, synchronous (gloo all-reduce) or
asynchronous (shared tensor over loopback TCP).  Prints one JSON line."""
import json
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import sharedtensor  # noqa: E402
from sharedtensor_b200.models import CharRNN, flatten_parameters  # noqa: E402
from sharedtensor_b200.parallel.trainers import AsyncTrainer, SyncTrainer, structured_token_batches  # noqa: E402


def main():
    rank, world, port, mode, steps = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3]), sys.argv[4], int(sys.argv[5])
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(7)  # every rank starts from the same weights
    model = CharRNN(vocab=13, hidden=24, layers=1)
    data = structured_token_batches(13, 8, 10, torch.device("cpu"), seed=10 + rank, period=1)
    shared = None
    if mode == "sync":
        # the mean of `world` gradients with step size world * lr is the sum the async replicas apply
        trainer = SyncTrainer(model, lr=0.3 * world)
    else:
        init, _ = flatten_parameters(model, align=32)
        for r in range(world):  # rank 0 founds the tensor, the others join it
            if r == rank:
                shared = sharedtensor.createOrFetch("127.0.0.1", port + 1, init)
            dist.barrier()
        trainer = AsyncTrainer(model, shared, lr=0.3)
    log = trainer.run(data, steps=steps, log_every=steps - 1)
    dist.barrier()
    checksum = None
    if shared is not None:
        shared.flush(10.0)
        dist.barrier()
        out = torch.empty(shared.numel)
        shared.copyToTensor(out)
        checksum = [float(out.double().sum()), float(out.double().norm())]
    print(json.dumps({"rank": rank, "mode": mode, "loss_first": log.loss[0], "loss_last": log.loss[-1], "checksum": checksum}), flush=True)
    dist.barrier()
    if shared is not None:
        time.sleep(0.2 * (world - rank))  # leaves first
        shared.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
