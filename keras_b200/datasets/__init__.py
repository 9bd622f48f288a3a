"""``keras.datasets``: small benchmark datasets downloaded on first use into ``~/.keras/datasets``."""

from keras_b200.datasets import boston_housing, california_housing, cifar10, cifar100, fashion_mnist, imdb, mnist, reuters  # noqa: F401
