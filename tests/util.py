import numpy as np

# Tolerances of the path (fp16/bf16 compute against the fp32 CPU reference), stated by the benchmark spec:
MAX_ABS_TOL = 2e-2      # max-abs error on the encoder output
COS_TOL = 0.9995        # cosine similarity over the whole tensor


def max_abs(a, b):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max())


def cosine(a, b):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    return float((a @ b) / np.sqrt((a @ a) * (b @ b)))


def valid_rows(arr, lengths):
    """Concatenate the valid (non-padded) positions of a [B, S, H] array."""
    return np.concatenate([arr[b, :int(n)] for b, n in enumerate(lengths)], axis=0)
