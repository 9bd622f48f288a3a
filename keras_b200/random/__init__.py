from keras_b200.random.random import (  # noqa: F401
    beta, binomial, categorical, dropout, gamma, normal, randint, shuffle, truncated_normal, uniform,
)
from keras_b200.random.seed_generator import SeedGenerator  # noqa: F401
