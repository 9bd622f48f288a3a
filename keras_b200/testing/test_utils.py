"""Synthetic classification data and parameter products for tests (keras/src/testing/test_utils.py)."""

import itertools

import numpy as np


def get_test_data(train_samples, test_samples, input_shape, num_classes, random_seed=None):
    """Gaussian clusters, one per class, split (stratified) into train and test parts."""
    rng = np.random.RandomState(random_seed)
    total = train_samples + test_samples
    per_class = total // num_classes
    extra = total % num_classes
    ys = np.array([i for i in range(num_classes) for _ in range(per_class)] + list(range(extra)), dtype=np.int32)
    templates = 2 * num_classes * rng.random((num_classes,) + tuple(input_shape))
    x = np.zeros((total,) + tuple(input_shape), dtype=np.float32)
    for i in range(total):
        x[i] = templates[ys[i]] + rng.normal(loc=0, scale=1.0, size=input_shape)
    order = rng.permutation(total)
    x, ys = x[order], ys[order]
    x_train, y_train, x_test, y_test = [], [], [], []
    for cls in range(num_classes):
        idx = np.where(ys == cls)[0]
        n_train = int(round(len(idx) * train_samples / total))
        x_train.append(x[idx[:n_train]])
        y_train.append(ys[idx[:n_train]])
        x_test.append(x[idx[n_train:]])
        y_test.append(ys[idx[n_train:]])
    x_train, y_train = np.concatenate(x_train), np.concatenate(y_train)
    x_test, y_test = np.concatenate(x_test), np.concatenate(y_test)
    p1, p2 = rng.permutation(len(x_train)), rng.permutation(len(x_test))
    return (x_train[p1], y_train[p1]), (x_test[p2], y_test[p2])


def named_product(*args, **kwargs):
    """``[{"testcase_name": ..., **params}]`` for every combination of the keyword lists (and named dict lists)."""
    def name_of(v):
        return str(v.__name__ if hasattr(v, "__name__") else v)

    groups = list(args)
    for key, values in kwargs.items():
        groups.append([{"testcase_name": f"{key}_{name_of(v)}", key: v} for v in values])
    out = []
    for combo in itertools.product(*groups):
        merged = {}
        names = []
        for d in combo:
            d = dict(d)
            names.append(d.pop("testcase_name"))
            merged.update(d)
        merged["testcase_name"] = "_".join(names)
        out.append(merged)
    return out
