"""CPU oracle for the quantized layer ops. TEST INFRASTRUCTURE ONLY: the product
package never imports this (see tosa_oracle.h for the parity status)."""
