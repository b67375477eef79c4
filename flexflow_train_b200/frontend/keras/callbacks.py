"""Keras-style callbacks (bindings/python/old/flexflow/keras/callbacks.py): hooks around training, a history
recorder, a learning-rate scheduler and the accuracy checks the legacy example scripts use."""


class Callback:
    def __init__(self):
        self.model = None

    def set_model(self, model):
        self.model = model

    def on_train_begin(self, logs=None): pass
    def on_train_end(self, logs=None): pass
    def on_epoch_begin(self, epoch, logs=None): pass
    def on_epoch_end(self, epoch, logs=None): pass
    def on_batch_begin(self, batch, logs=None): pass
    def on_batch_end(self, batch, logs=None): pass


class History(Callback):
    def on_train_begin(self, logs=None):
        self.epoch, self.history = [], {}

    def on_epoch_end(self, epoch, logs=None):
        self.epoch.append(epoch)
        for k, v in (logs or {}).items():
            self.history.setdefault(k, []).append(v)


class LearningRateScheduler(Callback):
    def __init__(self, schedule):
        super().__init__()
        self.schedule = schedule

    def on_epoch_begin(self, epoch, logs=None):
        opt = self.model.optimizer
        lr = self.schedule(epoch, opt.config.lr) if self.schedule.__code__.co_argcount > 1 else self.schedule(epoch)
        opt.set_learning_rate(lr)
        self.model.ffmodel.executable.cfg.optimizer.lr = lr


class VerifyMetrics(Callback):
    """Fails at the end of training when accuracy stayed under the target."""

    def __init__(self, accuracy):
        super().__init__()
        self.accuracy = getattr(accuracy, "value", accuracy)

    def on_train_end(self, logs=None):
        acc = 100.0 * (logs or {}).get("accuracy", 0.0)
        assert acc >= self.accuracy, f"accuracy {acc:.2f}% is below the target {self.accuracy}%"


class EpochVerifyMetrics(Callback):
    """Stops training early once the target accuracy is reached."""

    def __init__(self, accuracy, early_stop=True):
        super().__init__()
        self.accuracy = getattr(accuracy, "value", accuracy)
        self.early_stop = early_stop

    def on_epoch_end(self, epoch, logs=None):
        if self.early_stop and 100.0 * (logs or {}).get("accuracy", 0.0) >= self.accuracy:
            self.model.stop_training = True
