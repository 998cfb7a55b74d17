"""Whole-model launcher with the reference's command line (inference-engine/run_model.py:7-13):

    python run_model.py --transformer_config_file configs/vit_base_model.yaml
                        [--model_weight_file weights.npz] [--separate_qkv] [--need_compile] [--need_breakdown] [--tune]

layer_num encoder layers back to back (transformer_model.cpp:13-49).  Weights come from a
converted .npz checkpoint when the file exists, else random (test_transformer.cpp:470-489).  A checkpoint
written by weight_converter.py holds the three projections query / key / value, which run as three
operators - the reference builds this driver with -DSEPARATE=1 (run_model.py:130); --separate_qkv asks
for that form with random weights too.
"""
import run_layer

if __name__ == '__main__':
    run_layer.run(run_layer.parse_args(), whole_model=True)
