from keras_b200.optimizers.schedules.learning_rate_schedule import (  # noqa: F401
    CosineDecay, CosineDecayRestarts, ExponentialDecay, InverseTimeDecay, LearningRateSchedule,
    PiecewiseConstantDecay, PolynomialDecay, deserialize, serialize,
)
