class WeightError(ValueError):
    """The tensors of a model file do not match what the model needs.

    `missing`, `unexpected` and `wrong_shape` list all faults found, so one
    failed load names everything that has to be fixed."""

    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=()):
        super().__init__(message)
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)
        self.wrong_dtype = list(wrong_dtype)
