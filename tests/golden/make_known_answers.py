"""Writes reference_known_answers.json: the known-answer vectors that the reference's own
tests assert for this path and that do not depend on JAX's PRNG stream.

The reference is Python-on-JAX and JAX cannot be installed where this repository is built,
so the vectors are transcribed from the reference's test files (cited per entry, paths
inside the google/qwix tree) rather than produced by running it.

  python tests/golden/make_known_answers.py
"""

import json
import pathlib

INF = 'inf'

VECTORS = {
    'convert_to': [
        # tests/_src/core/numerics_test.py:34-50
        {'src': 'numerics_test.py:35-41', 'qtype': 'int8',
         'x': [1.2, 3.5, -127.5, 129, -1300], 'want': [1, 4, -128, 127, -128]},
        {'src': 'numerics_test.py:42-45', 'qtype': 'int4',
         'x': [1.2, 3.5, 8, -1300], 'want': [1, 4, 7, -8]},
        {'src': 'numerics_test.py:46-50', 'qtype': 'int16',
         'x': [1.2, 3.5, -32768.5, 32769, -40000], 'want': [1, 4, -32768, 32767, -32768]},
        # numerics_test.py:52-56
        {'src': 'numerics_test.py:52-56', 'qtype': 'int8', 'x': [INF, '-inf'],
         'want': [127, -128]},
        # numerics_test.py:58-88
        {'src': 'numerics_test.py:60-63', 'qtype': 'int6',
         'x': [1.2, 3.5, 129, -1300], 'want': [1, 4, 31, -32]},
        {'src': 'numerics_test.py:84-88', 'qtype': 'uint8',
         'x': [-1.2, 3.5, 129, 1300], 'want': [0, 4, 129, 255]},
        # numerics_test.py:108-112
        {'src': 'numerics_test.py:109-112', 'qtype': 'nf4',
         'x': [-1.0, -0.5, 0.0, 0.8, 1.0], 'want': [0, 2, 7, 14, 15]},
        # numerics_test.py:133-189 (values after conversion back to float)
        {'src': 'numerics_test.py:133-145', 'qtype': 'mxfp8',
         'x': [10.0, 500.0, -1000.0], 'want': [10.0, 448.0, -448.0]},
        {'src': 'numerics_test.py:152-164', 'qtype': 'mxfp8_16',
         'x': [10.0, 500.0, -1000.0], 'want': [10.0, 448.0, -448.0]},
        {'src': 'numerics_test.py:176-184', 'qtype': 'mxfp4',
         'x': [1.5, 10.0, -20.0], 'want': [1.5, 6.0, -6.0]},
        {'src': 'numerics_test.py:186-193', 'qtype': 'nvfp4',
         'x': [1.5, 10.0, -20.0], 'want': [1.5, 6.0, -6.0]},
    ],
    'symmetric_bound': [
        {'src': 'numerics_test.py:59', 'qtype': 'int6', 'want': 31.5},
        {'src': 'numerics_test.py:64', 'qtype': 'int16', 'want': 32768.0},
        {'src': 'numerics_test.py:85', 'qtype': 'uint8', 'want': 255.5},
        {'src': 'numerics_test.py:129-131', 'qtype': 'mxfp8', 'want': 448.0},
        {'src': 'numerics_test.py:166-169', 'qtype': 'mxfp4', 'want': 6.0},
        {'src': 'numerics_test.py:171-174', 'qtype': 'nvfp4', 'want': 6.0},
        {'src': 'qwix/_src/core/numerics.py:134-136', 'qtype': 'int8', 'want': 127.5},
        {'src': 'qwix/_src/core/numerics.py:134-136', 'qtype': 'int4', 'want': 7.5},
        {'src': 'qwix/_src/core/numerics.py:132', 'qtype': 'float8_e4m3fn', 'want': 448.0},
    ],
    'nf4_convert_from': {'src': 'numerics_test.py:113-116', 'codes': [0, 7, 15],
                         'want': [-1.0, 0.0, 1.0]},
    # tests/_src/core/qarray_test.py:191-219 (without_error): 0..255/255, int8 minmax.
    'exact_minmax_round_trip': {'src': 'qarray_test.py:191-219', 'count': 256,
                                'zero_point': -128, 'first_code': -128, 'last_code': 127},
    # qarray_test.py:221-226
    'get_tiled_axes': {'src': 'qarray_test.py:221-226', 'qvalue_shape': [10, 256, 16],
                       'scale_shape': [10, 8, 2], 'want': {'1': 32, '2': 8}},
    # qarray_test.py:228-302: shapes of the scale under reshape / transpose / slicing of a
    # (2, 2, 6) array quantized with channelwise axis 0 and tile 2 on axis 2.
    'array_methods': {
        'src': 'qarray_test.py:228-302', 'shape': [2, 2, 6], 'channelwise_axes': [0],
        'tiled_axes': {'2': 2}, 'scale_shape': [2, 1, 3], 'scale_tile_shape': [1, 2, 2],
        'reshape': [[[4, 1, 3, 2], [2, 1, 3, 1]], [[2, 1, 2, 6], [2, 1, 1, 3]],
                    [[1, 4, 6], [1, 2, 3]]],
        'reshape_chain': {'first': [4, 1, 3, 2], 'then': [4, 6], 'scale_shape': [2, 3]},
        'transpose': [[[1, 2, 0], [2, 6, 2], [1, 3, 2]]],
        'T': [[6, 2, 2], [3, 1, 2]], 'mT': [[2, 6, 2], [2, 3, 1]],
        'swapaxes_1_2': [[2, 6, 2], [2, 3, 1]],
    },
    # qarray_test.py:505-532: outlier-aware power-of-two scales.
    'mxfp_scales': [
        {'src': 'qarray_test.py:507-512', 'qtype': 'mxfp4', 'absmax': [6.5, 7.5], 'want': [1.0, 2.0]},
        {'src': 'qarray_test.py:513-518', 'qtype': 'mxfp8', 'absmax': [460.0, 465.0], 'want': [1.0, 2.0]},
        {'src': 'qarray_test.py:519-524', 'qtype': 'mxfp8_16', 'absmax': [460.0, 465.0], 'want': [1.0, 2.0]},
    ],
    # tests/_src/core/pallas_test.py:39-88: block shape / index map of the scale.
    'pallas_block_specs': [
        {'src': 'pallas_test.py:41-47', 'block_shape': [128, 128], 'qvalue_shape': [1024, 1024],
         'scale_shape': [1024, 1], 'scale_block_shape': [128, 1], 'index': [1, 1], 'scale_index': [1, 0]},
        {'src': 'pallas_test.py:49-55', 'block_shape': [256, 256], 'qvalue_shape': [1024, 1024],
         'scale_shape': [32, 8], 'scale_block_shape': [8, 2], 'index': [1, 1], 'scale_index': [1, 1]},
        {'src': 'pallas_test.py:57-63', 'block_shape': [None, 256], 'qvalue_shape': [1024, 1024],
         'scale_shape': [1024, 8], 'scale_block_shape': [None, 2], 'index': [1, 1], 'scale_index': [1, 1]},
    ],
    # tests/_src/providers/ptq_test.py:36-86: Dense 12 -> 5 with tile_size 4.
    'ptq_dense_tile': {'src': 'ptq_test.py:36-86', 'kernel_shape': [12, 5], 'tile_size': 4,
                       'scale_shape': [3, 5]},
    # tests/contrib/hadamard_rot_test.py:31-44: H H^T = d I.
    'hadamard_orthogonality': {'src': 'hadamard_rot_test.py:31-44', 'powers': [1, 3, 7]},
}

if __name__ == '__main__':
  out = pathlib.Path(__file__).with_name('reference_known_answers.json')
  out.write_text(json.dumps(VECTORS, indent=1) + '\n')
  print(out)
