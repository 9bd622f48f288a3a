"""``keras.export``: serving artefacts.

The reference exports through TensorFlow SavedModel, tf2onnx / ``torch.onnx``, LiteRT and OpenVINO
(keras/src/export/*.py).  This framework has one tensor runtime, so the native artefact is a ``torch.export``
program archive (``format="torch_export"``: one ``.pt2`` per endpoint plus a JSON manifest); ONNX goes through
``torch.onnx`` when the ``onnx`` package is installed, and the TensorFlow-, LiteRT- and OpenVINO-based formats raise an
``ImportError`` naming the missing runtime.
"""

from keras_b200.export.export_archive import ExportArchive, export_model, load_exported  # noqa: F401
