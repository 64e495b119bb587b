"""Seeded synthetic inputs for the prediction path.

The reference ships neither traces nor trained checkpoints, so benchmarks and
parity tests draw their inputs here.  Value ranges follow the grids the
reference samples when it collects MLP training data
(tools/recording/record_linear.py:72-74, record_conv2d.py:121-128,
record_bmm.py:53-56, record_lstm.py:79-83) and typical CUDA launch shapes.
Everything is a pure function of the seed (numpy PCG64).
"""
import numpy as np

# The six destination rows of the synthetic benchmark, in order.
BENCH_DEVICES = ("V100_16", "V100_32", "A100_40", "H100_80", "RTX3090", "B200")

# (mem GB, mem_bw GB/s, num_sm, fp32 TFLOP/s): MLP device features per row
BENCH_DEVICE_FEATURES = np.array([
    (16, 900, 80, 15.7), (32, 900, 80, 15.7), (40, 1555, 108, 19.5),
    (80, 3350, 132, 67), (24, 936, 82, 35.6), (180, 8000, 148, 80)], dtype=np.float64)

OP_FEATURES = {
    "linear": ["bias", "batch", "in_features", "out_features"],
    "lstm": ["bias", "bidirectional", "batch", "seq_len", "input_size", "hidden_size", "num_layers"],
    "conv2d": ["bias", "batch", "image_size", "in_channels", "out_channels", "kernel_size",
               "stride", "padding"],
    "bmm": ["batch", "left", "middle", "right"],
}
WEIGHT_SEED = {"linear": 0, "conv2d": 1, "bmm": 2, "lstm": 3}


def rng(seed):
    return np.random.Generator(np.random.PCG64(seed))


def log_uniform_int(g, lo, hi, n):
    """Integers in [lo, hi] with log-uniform density."""
    u = g.uniform(np.log(lo), np.log(hi + 1), size=n)
    return np.clip(np.floor(np.exp(u)), lo, hi).astype(np.int64)


def make_kernels(n, seed, valid_only=False, origin=None):
    """n recorded kernels: grid blocks LU[1, 2^20], block size from {32..1024},
    registers U[16, 255], shared memory 256 B * U[0, 384], time LU[2e3, 5e7] ns,
    gamma U[0, 1].  valid_only rejection-samples to origin occupancy > 0 (needs
    `origin`, a function (block, smem, regs) -> occupancy array)."""
    g = rng(seed)

    def draw(m):
        return dict(
            num_blocks=log_uniform_int(g, 1, 1 << 20, m).astype(np.int32),
            block_size=g.choice(np.array([32, 64, 128, 256, 512, 1024]), size=m).astype(np.uint16),
            regs_per_thread=g.integers(16, 256, size=m).astype(np.uint16),
            smem_bytes=(256 * g.integers(0, 385, size=m)).astype(np.uint32),
            run_time_ns=log_uniform_int(g, 2000, 50_000_000, m).astype(np.float64),
            gamma=g.uniform(0.0, 1.0, size=m).astype(np.float32),
        )

    if not valid_only:
        return draw(n)
    parts, have = [], 0
    while have < n:
        d = draw(max(1024, 3 * (n - have)))
        keep = origin(d["block_size"], d["smem_bytes"], d["regs_per_thread"]) > 0
        d = {k: v[keep] for k, v in d.items()}
        parts.append(d)
        have += len(d["num_blocks"])
    return {k: np.concatenate([p[k] for p in parts])[:n] for k in parts[0]}


def make_metrics(n, seed):
    """Raw metrics for the kernels of make_kernels: SP FLOP efficiency (%), DRAM
    bytes read / written, and a has-metrics flag (about one kernel in eight has
    none; a few have zero traffic or zero FLOPs to hit the special cases)."""
    g = rng(seed)
    eff = g.uniform(0.0, 80.0, size=n)
    rd = np.floor(np.exp(g.uniform(np.log(1e3), np.log(1e10), size=n)))
    wr = np.floor(np.exp(g.uniform(np.log(1e3), np.log(1e10), size=n)))
    kind = g.integers(0, 32, size=n)
    eff[kind == 0] = 0.0
    rd[kind == 1] = 0.0
    wr[kind == 1] = 0.0
    has = (g.integers(0, 8, size=n) != 0).astype(np.uint8)
    return dict(flop_efficiency_pct=eff, dram_read_bytes=rd, dram_write_bytes=wr, has_metrics=has)


def make_queries(op, n, seed):
    """[n, F] float32 op features and [n] uint8 device rows (uniform over the six)."""
    g = rng(seed)
    if op == "linear":
        cols = [g.integers(0, 2, n), log_uniform_int(g, 1, 3500, n),
                log_uniform_int(g, 1, 32768, n), log_uniform_int(g, 1, 32768, n)]
    elif op == "conv2d":
        cols = [g.integers(0, 2, n), log_uniform_int(g, 1, 64, n), log_uniform_int(g, 1, 256, n),
                log_uniform_int(g, 3, 2048, n), log_uniform_int(g, 3, 2048, n),
                g.choice(np.array([1, 3, 5, 7]), size=n), g.choice(np.array([1, 2, 4]), size=n),
                g.integers(0, 4, n)]
    elif op == "bmm":
        cols = [log_uniform_int(g, 1, 512, n)] + [log_uniform_int(g, 1, 4096, n) for _ in range(3)]
    elif op == "lstm":
        cols = [g.integers(0, 2, n), g.integers(0, 2, n), log_uniform_int(g, 1, 128, n),
                log_uniform_int(g, 1, 512, n), log_uniform_int(g, 32, 4096, n),
                log_uniform_int(g, 32, 4096, n), g.integers(1, 5, n)]
    else:
        raise ValueError(op)
    feats = np.stack(cols, axis=1).astype(np.float32)
    dev = g.integers(0, len(BENCH_DEVICES), n).astype(np.uint8)
    return feats, dev


def batch_mu_sigma(feats, dev_rows, device_features=BENCH_DEVICE_FEATURES):
    """mean / population std of the [n, F+4] feature matrix (the rule of the
    reference's training set, analysis/mlp/dataset.py:16-19)."""
    x = np.concatenate([feats.astype(np.float64), device_features[dev_rows]], axis=1)
    sigma = x.std(axis=0)
    sigma[sigma == 0] = 1.0
    return x.mean(axis=0), sigma


def init_mlp_weights(op, seed=None, layers=8, width=1024, gain=1.0):
    """Random-init weights with torch.nn.Linear's default distribution
    (uniform +-1/sqrt(fan_in)), drawn with numpy so no torch is needed.
    gain scales fc1 and hidden weights (sqrt(6) keeps activation variance, which
    makes outputs depend visibly on inputs)."""
    g = rng(WEIGHT_SEED[op] if seed is None else seed)
    F = len(OP_FEATURES[op])

    def lin(out_f, in_f, scale=1.0):
        b = 1.0 / np.sqrt(in_f)
        return ((g.uniform(-b, b, size=(out_f, in_f)) * scale).astype(np.float32),
                g.uniform(-b, b, size=(out_f,)).astype(np.float32))

    fc1_w, fc1_b = lin(width, F + 4, gain)
    hw, hb = zip(*[lin(width, width, gain) for _ in range(layers)])
    fc2_w, fc2_b = lin(1, width)
    return dict(fc1_w=fc1_w, fc1_b=fc1_b, hidden_w=np.stack(hw), hidden_b=np.stack(hb),
                fc2_w=fc2_w.reshape(-1), fc2_b=fc2_b)


def torch_init_mlp_weights(op, seed=None, layers=8, width=1024):
    """Weights exactly as the reference creates them for a fresh predictor:
    torch.manual_seed(seed) followed by the construction of the op's MLP class
    (torch.nn.Linear default init, modules created in the order fc1, hidden
    stack, fc2 as in analysis/mlp/mlp.py:34-50)."""
    import torch
    from habitat_b200.analysis.mlp.mlp import RuntimePredictor, state_to_arrays
    state = torch.random.get_rng_state()
    try:
        torch.manual_seed(WEIGHT_SEED[op] if seed is None else seed)
        pred = RuntimePredictor(op, layers, width)
    finally:
        torch.random.set_rng_state(state)
    return state_to_arrays(pred.model)


# ---------------------------------------------------------------------------
# The fixed batch of the scale sweep: 67,108,864 (kernel, destination) pairs rounded up to whole
# kernels and to an even number of them = 11,184,812 kernels x 6 destinations (eight pairs of
# padding; an even count keeps every output plane on an 8-byte boundary) and 4,194,304 queries
# for each of the four predictors.  Records are generated in chunks of 262,144 from per-chunk seeds,
# so any rank can produce exactly its shard [lo, hi) without generating the rest.
# ---------------------------------------------------------------------------
SWEEP_KERNELS = 11_184_812
SWEEP_QUERIES = 4_194_304
SWEEP_OPS = ("conv2d", "linear", "bmm", "lstm")
SWEEP_CHUNK = 1 << 18


def _chunked(lo, hi, make):
    """Concatenates make(chunk index) over the chunks that overlap [lo, hi) and cuts to it."""
    parts = []
    for c in range(lo // SWEEP_CHUNK, (max(hi, lo + 1) - 1) // SWEEP_CHUNK + 1):
        part = make(c)
        a = max(lo - c * SWEEP_CHUNK, 0)
        b = min(hi - c * SWEEP_CHUNK, SWEEP_CHUNK)
        parts.append(tuple(x[a:b] for x in part))
    return [np.concatenate([p[i] for p in parts]) for i in range(len(parts[0]))]


def sweep_kernels(lo, hi, seed=5000):
    """Records [lo, hi) of the sweep's kernel batch (same fields as make_kernels)."""
    names = ("num_blocks", "block_size", "regs_per_thread", "smem_bytes", "run_time_ns", "gamma")
    cols = _chunked(lo, hi, lambda c: tuple(make_kernels(SWEEP_CHUNK, seed + c)[n] for n in names))
    return dict(zip(names, cols))


def sweep_queries(op, lo, hi, seed=6000):
    """Queries [lo, hi) of the sweep's batch for predictor `op`: ([n, F] float32, [n] uint8)."""
    base = seed + 1000 * SWEEP_OPS.index(op)
    feats, dev = _chunked(lo, hi, lambda c: make_queries(op, SWEEP_CHUNK, base + c))
    return feats, dev


def sweep_mu_sigma(op, seed=6000):
    """Normalisation of the sweep's predictor `op`: mean / population std over the first chunk
    of its batch (every rank computes the same values without seeing the whole batch)."""
    feats, dev = sweep_queries(op, 0, SWEEP_CHUNK, seed)
    return batch_mu_sigma(feats, dev)


# ---------------------------------------------------------------------------
# The mixed iteration trace: every iteration holds 53 conv2d, 1 linear and 32 bmm operations
# predicted by their MLPs and 74 ordinary operations of one wave-scaled kernel each.
# ---------------------------------------------------------------------------
ITER_SPECIAL = {"conv2d": 53, "linear": 1, "bmm": 32}
ITER_KERNELS = 74


def make_iterations(lo, hi, origin_occupancy, seed=4000):
    """Iterations [lo, hi) of the mixed trace, generated per iteration from its own seed.
    origin_occupancy(block, smem, regs) -> occupancy array on the origin (kernels are
    rejection-sampled so that the origin can run them).  Returns (kernels dict, overhead_ns
    float32 [n * 74], {op: (features, measured ms)})."""
    ks, over, ops = [], [], {op: ([], []) for op in ITER_SPECIAL}
    for it in range(lo, hi):
        ks.append(make_kernels(ITER_KERNELS, seed + 10 * it, valid_only=True, origin=origin_occupancy))
        g = rng(seed + 10 * it + 1)
        over.append(g.uniform(0, 10_000, size=ITER_KERNELS).astype(np.float32))
        for j, (op, n) in enumerate(ITER_SPECIAL.items()):
            feats, _ = make_queries(op, n, seed + 10 * it + 2 + j)
            ops[op][0].append(feats)
            ops[op][1].append(np.exp(g.uniform(np.log(0.02), np.log(50.0), size=n)).astype(np.float32))
    kernels = {k: np.concatenate([x[k] for x in ks]) for k in ks[0]} if ks else make_kernels(0, seed)
    special = {op: (np.concatenate(f) if f else np.zeros((0, len(OP_FEATURES[op])), np.float32),
                    np.concatenate(t) if t else np.zeros(0, np.float32)) for op, (f, t) in ops.items()}
    return kernels, (np.concatenate(over) if over else np.zeros(0, np.float32)), special
